// Reading and writing safetensors files through a memory mapping.
//
// File layout: an 8-byte little-endian header length, a JSON header that maps tensor names to
// {"dtype", "shape", "data_offsets"} with offsets relative to the end of the header, then the data.  A model
// folder holds either model.safetensors or model.safetensors.index.json whose "weight_map" names the shard of
// every tensor.  The reference's reader does the same over an mmap (src/safetensors_mmap.cpp:213-256 for a
// shard: header longer than the file :225, bad dtype / shape entries :236-239, tensor outside the file :246,
// duplicate across shards :250, "__metadata__" skipped :233; :260-287 for a folder, shards in order of first
// appearance :269-279).
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../host/common.h"
#include "../host/json.h"

namespace qe {

struct TensorEntry {
    std::string name;
    DType dtype = DType::F32;
    std::string dtype_name;               // as the file spells it ("BF16", "F32", ...)
    std::vector<int64_t> shape;
    const uint8_t* data = nullptr;        // inside the mapping
    size_t bytes = 0;
    int64_t numel() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
};

class QE_API SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;
    const std::string& path() const { return path_; }
    const std::vector<TensorEntry>& entries() const { return entries_; }
    const Json& metadata() const { return metadata_; }
private:
    std::string path_;
    int fd_ = -1;
    uint8_t* map_ = nullptr;
    size_t size_ = 0;
    std::vector<TensorEntry> entries_;
    Json metadata_;
};

// All tensors of a model folder, whatever shard they are in.
class QE_API SafetensorsFolder {
public:
    explicit SafetensorsFolder(const std::string& model_dir);
    const std::string& model_dir() const { return dir_; }
    std::vector<std::string> names() const;                       // in file order
    const TensorEntry* find(const std::string& name) const;
    const TensorEntry& at(const std::string& name) const;
private:
    std::string dir_;
    std::vector<std::unique_ptr<SafetensorsFile>> files_;
    std::vector<std::string> order_;
    std::map<std::string, const TensorEntry*> by_name_;
};

// One tensor to write: its bytes are produced by `fill(dst)` when its turn comes, so that a large model never
// sits in memory whole.
struct TensorToWrite {
    std::string name;
    DType dtype;
    std::vector<int64_t> shape;
    std::function<void(uint8_t* dst)> fill;
};
QE_API void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors, const Json& metadata);

QE_API DType safetensors_dtype(const std::string& name, bool* ok);
QE_API const char* safetensors_dtype_name(DType d);

}  // namespace qe

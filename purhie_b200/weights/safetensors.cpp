#include "safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <fstream>
#include <sstream>

namespace qe {

namespace {
struct DTypeName { const char* name; DType dtype; };
const DTypeName kDTypes[] = {{"F64", DType::F64}, {"F32", DType::F32}, {"F16", DType::F16}, {"BF16", DType::BF16},
                             {"I64", DType::I64}, {"I32", DType::I32}, {"I16", DType::I16}, {"I8", DType::I8},
                             {"U8", DType::U8},   {"BOOL", DType::BOOL}};

bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0;
}
std::string read_text(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw SafetensorsError(path + ": cannot open (" + strerror(errno) + ")");
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
}  // namespace

DType safetensors_dtype(const std::string& name, bool* ok) {
    for (const auto& d : kDTypes)
        if (name == d.name) { *ok = true; return d.dtype; }
    *ok = false;
    return DType::F32;
}
const char* safetensors_dtype_name(DType d) {
    for (const auto& e : kDTypes)
        if (e.dtype == d) return e.name;
    return "?";
}

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = open(path.c_str(), O_RDONLY);
    if (fd_ < 0) throw SafetensorsError(path + ": cannot open (" + strerror(errno) + ")");
    struct stat st;
    if (fstat(fd_, &st) != 0) { close(fd_); throw SafetensorsError(path + ": cannot stat"); }
    size_ = (size_t)st.st_size;
    auto fail = [&](const std::string& what) {
        if (map_) munmap(map_, size_);
        close(fd_);
        map_ = nullptr; fd_ = -1;
        throw SafetensorsError(path + ": " + what);
    };
    if (size_ < 8) fail("too short to hold a header length (" + std::to_string(size_) + " bytes)");
    void* m = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (m == MAP_FAILED) { map_ = nullptr; fail(std::string("cannot map (") + strerror(errno) + ")"); }
    map_ = static_cast<uint8_t*>(m);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | map_[i];
    if (hlen > size_ || 8 + hlen > size_)
        fail("header of " + std::to_string(hlen) + " bytes is longer than the file (" + std::to_string(size_) + " bytes)");
    Json header;
    try {
        header = Json::parse(reinterpret_cast<const char*>(map_ + 8), (size_t)hlen);
    } catch (const JsonError& e) {
        fail(std::string("header is not valid JSON (") + e.what() + ")");
    }
    if (!header.is_object()) fail("header must be a JSON object");
    const size_t data_start = 8 + (size_t)hlen;
    for (const auto& m2 : header.members()) {
        const std::string& name = m2.first;
        const Json& info = m2.second;
        if (name == "__metadata__") { metadata_ = info; continue; }
        const Json *jd = info.find("dtype"), *js = info.find("shape"), *jo = info.find("data_offsets");
        if (!jd || !js || !jo || !jd->is_string() || !js->is_array() || !jo->is_array() || jo->size() != 2)
            fail("tensor '" + name + "' has a malformed entry");
        bool ok = false;
        TensorEntry e;
        e.name = name;
        e.dtype_name = jd->as_string();
        e.dtype = safetensors_dtype(e.dtype_name, &ok);
        if (!ok) fail("tensor '" + name + "' has unsupported dtype '" + e.dtype_name + "'");
        int64_t n = 1;
        for (const Json& s : js->items()) {
            if (!s.is_int() || s.as_int() < 0) fail("tensor '" + name + "' has a malformed shape " + js->dump());
            e.shape.push_back(s.as_int());
            n *= s.as_int();
        }
        if (!(*jo)[0].is_int() || !(*jo)[1].is_int()) fail("tensor '" + name + "' has malformed offsets");
        long long b = (*jo)[0].as_int(), en = (*jo)[1].as_int();
        if (b < 0 || en < b || (uint64_t)(en - b) != (uint64_t)n * dtype_size(e.dtype))
            fail("tensor '" + name + "': offsets [" + std::to_string(b) + ", " + std::to_string(en) +
                 ") do not match shape " + shape_text(e.shape) + " of " + e.dtype_name);
        if (data_start + (size_t)en > size_)
            fail("tensor '" + name + "' ends at byte " + std::to_string(data_start + (size_t)en) + ", the file has " +
                 std::to_string(size_));
        e.data = map_ + data_start + (size_t)b;
        e.bytes = (size_t)(en - b);
        entries_.push_back(std::move(e));
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_) munmap(map_, size_);
    if (fd_ >= 0) close(fd_);
}

SafetensorsFolder::SafetensorsFolder(const std::string& model_dir) : dir_(model_dir) {
    const std::string index = model_dir + "/model.safetensors.index.json", single = model_dir + "/model.safetensors";
    auto add = [&](const std::string& path) {
        files_.emplace_back(new SafetensorsFile(path));
        for (const TensorEntry& e : files_.back()->entries()) {
            auto it = by_name_.find(e.name);
            if (it != by_name_.end()) {
                std::string other;
                for (const auto& f : files_)
                    for (const TensorEntry& o : f->entries())
                        if (&o == it->second) other = f->path();
                throw SafetensorsError("tensor '" + e.name + "' is in both " + other + " and " + path);
            }
            by_name_[e.name] = &e;
            order_.push_back(e.name);
        }
    };
    if (file_exists(index)) {
        Json idx;
        const Json* wm = nullptr;
        try {
            idx = Json::parse(read_text(index));
            wm = idx.find("weight_map");
        } catch (const JsonError& e) {
            throw SafetensorsError(index + ": no usable 'weight_map' (" + e.what() + ")");
        }
        if (!wm || !wm->is_object()) throw SafetensorsError(index + ": no usable 'weight_map'");
        std::vector<std::string> shards;
        for (const auto& m : wm->members()) {
            if (!m.second.is_string()) throw SafetensorsError(index + ": no usable 'weight_map' (a shard name is not a string)");
            bool seen = false;
            for (const auto& s : shards) seen |= (s == m.second.as_string());
            if (!seen) shards.push_back(m.second.as_string());
        }
        for (const auto& s : shards) add(model_dir + "/" + s);
        for (const auto& m : wm->members())
            if (!by_name_.count(m.first))
                throw SafetensorsError(index + ": tensor '" + m.first + "' is not in " + m.second.as_string());
    } else if (file_exists(single)) {
        add(single);
    } else {
        throw SafetensorsError(model_dir + ": neither model.safetensors nor model.safetensors.index.json");
    }
}

std::vector<std::string> SafetensorsFolder::names() const { return order_; }
const TensorEntry* SafetensorsFolder::find(const std::string& name) const {
    auto it = by_name_.find(name);
    return it == by_name_.end() ? nullptr : it->second;
}
const TensorEntry& SafetensorsFolder::at(const std::string& name) const {
    const TensorEntry* e = find(name);
    if (!e) throw SafetensorsError(dir_ + ": no tensor '" + name + "'");
    return *e;
}

void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors, const Json& metadata) {
    Json header = Json::object();
    if (metadata.is_object() && metadata.size()) header.set("__metadata__", metadata);
    size_t offset = 0, largest = 0;
    for (const auto& t : tensors) {
        if (header.has(t.name)) throw SafetensorsError(path + ": tensor '" + t.name + "' is listed twice");
        size_t n = 1;
        Json shape = Json::array();
        for (auto s : t.shape) { n *= (size_t)s; shape.push((long long)s); }
        size_t bytes = n * dtype_size(t.dtype);
        Json e = Json::object();
        e.set("dtype", safetensors_dtype_name(t.dtype));
        e.set("shape", shape);
        Json off = Json::array();
        off.push((long long)offset);
        off.push((long long)(offset + bytes));
        e.set("data_offsets", off);
        header.set(t.name, e);
        offset += bytes;
        largest = std::max(largest, bytes);
    }
    std::string blob = header.dump();
    blob.append((64 - (8 + blob.size()) % 64) % 64, ' ');          // the data starts on a 64-byte boundary
    const std::string tmp = path + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) throw SafetensorsError(tmp + ": cannot write (" + strerror(errno) + ")");
    uint8_t len[8];
    uint64_t hl = blob.size();
    for (int i = 0; i < 8; i++) len[i] = (uint8_t)(hl >> (8 * i));
    bool ok = fwrite(len, 1, 8, f) == 8 && fwrite(blob.data(), 1, blob.size(), f) == blob.size();
    std::vector<uint8_t> buf(largest);
    for (const auto& t : tensors) {
        if (!ok) break;
        size_t n = 1;
        for (auto s : t.shape) n *= (size_t)s;
        size_t bytes = n * dtype_size(t.dtype);
        if (bytes) {
            t.fill(buf.data());
            ok = fwrite(buf.data(), 1, bytes, f) == bytes;
        }
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) { unlink(tmp.c_str()); throw SafetensorsError(tmp + ": write failed (" + strerror(errno) + ")"); }
    if (rename(tmp.c_str(), path.c_str()) != 0) throw SafetensorsError(path + ": cannot replace (" + strerror(errno) + ")");
}

}  // namespace qe

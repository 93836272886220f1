// Loading a model's tensors by name, with one error for everything that does not fit; and seeded random weights.
//
// Every part of a model announces the tensors it needs as TensorSpec (name, shape, role).  The loader checks the
// whole folder against the whole list before it copies anything and raises one WeightError that lists missing
// tensors, unexpected tensors, wrong shapes and wrong types together.  The reference binds tensors one at a time
// and stops at the first problem (bind_weight src/inference.cpp:362-389, bind_norm :392-407, check_shape
// :426-430, "missing tensor" :365).
//
// Storage on the device:
//   role matrix: the compute dtype.  With compute dtype bfloat16 a tensor stored as BF16 stays BF16, F16 is
//     converted to BF16, and a tensor stored in 32-bit stays in 32-bit (the linear part then multiplies it with
//     the 32-bit kernel).  With compute dtype float32 everything is widened to float32.
//   role vector (norm weights, biases): float32 always; widening BF16 is exact.
//   role table (integer tables): int32.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../config/config.h"
#include "../parts/parts.h"
#include "safetensors.h"

namespace qe {

// How random weights are drawn: matrices N(0, std); norm weights U(scale_low, scale_high) (the constant when
// both are equal).  stored_dtype: how a matrix is stored before the dtype policy applies (a folder written as
// float32 keeps float32 matrices even in a bfloat16 run).
struct RandomInit {
    uint64_t seed = 0;
    double std = 0.02, scale_low = 1.0, scale_high = 1.0;
};

QE_API DType device_dtype(DType stored, Role role, DType compute);

// Check `folder` against `expected`; throws one WeightError listing everything that does not fit.
QE_API void check_folder(const SafetensorsFolder& folder, const std::vector<TensorSpec>& expected,
                         const std::vector<std::string>& ignore);

// Tensors from a checkpoint folder (checked against `expected` when constructed).
class QE_API FolderSource : public WeightSource {
public:
    FolderSource(const std::string& model_dir, const std::vector<TensorSpec>& expected, const std::vector<std::string>& ignore,
                 DType compute, DeviceArena& arena, cudaStream_t stream);
    Tensor fetch(const std::string& name) override;
    DeviceArena& arena() override { return arena_; }
    cudaStream_t stream() override { return stream_; }
private:
    SafetensorsFolder folder_;
    std::map<std::string, TensorSpec> specs_;
    std::map<std::string, Tensor> cache_;
    DType compute_;
    DeviceArena& arena_;
    cudaStream_t stream_;
};

// Tensors drawn on the device by the seeded generator (weights/random.h): the values a folder written by
// write_random_model with the same seed holds.
class QE_API RandomSource : public WeightSource {
public:
    RandomSource(const std::vector<TensorSpec>& expected, const RandomInit& init, DType stored_matrix_dtype, DType compute,
                 DeviceArena& arena, cudaStream_t stream);
    Tensor fetch(const std::string& name) override;
    DeviceArena& arena() override { return arena_; }
    cudaStream_t stream() override { return stream_; }
private:
    std::map<std::string, TensorSpec> specs_;
    std::map<std::string, Tensor> cache_;
    RandomInit init_;
    DType stored_, compute_;
    DeviceArena& arena_;
    cudaStream_t stream_;
};

// The tensors a model of this configuration reads, from its parts (built without a device).
QE_API std::vector<TensorSpec> expected_tensors(const ModelConfig& config);

// One tensor's random values on the host, as float32 (what a folder stores after rounding to its dtype).
QE_API std::vector<float> random_tensor_host(const TensorSpec& spec, const RandomInit& init);

// Write config.json and model.safetensors into model_dir.  matrix_dtype / vector_dtype: BF16, F16 or F32.
QE_API void write_random_model(const std::string& model_dir, const ModelConfig& config, const RandomInit& init,
                               DType matrix_dtype, DType vector_dtype);

}  // namespace qe

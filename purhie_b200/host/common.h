// What every part of the host library shares: error types, element types and the tensor view.
//
// Errors are C++ exceptions inside the library; the C API turns them into the codes of inference.h and keeps
// the text for inference_get_last_error().  A Tensor is a view (pointer, element type, shape) of device or host
// memory that somebody else owns: the model owns weights, the cache manager pools, a Workspace scratch.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#if defined(__GNUC__)
#define QE_API __attribute__((visibility("default")))
#else
#define QE_API
#endif

namespace qe {

// ---- errors ---------------------------------------------------------------------------------------------
// Codes are those of the C API (api/inference.h).
enum ErrorCode {
    kOk = 0, kInvalidArg = -1, kOutOfMemory = -2, kModelLoad = -3, kKvCache = -4, kKernelLaunch = -6,
    kInvalidState = -7, kNotImplemented = -8, kContextFull = -9, kCancelled = -10,
};

struct QE_API Error : std::runtime_error {
    int code;
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};
// A config.json that cannot be used: a missing key, a wrong type, an unsupported option, an unknown architecture.
struct QE_API ConfigError : Error { explicit ConfigError(const std::string& w) : Error(kModelLoad, w) {} };
// A file that is not a well-formed safetensors file or folder.
struct QE_API SafetensorsError : Error { explicit SafetensorsError(const std::string& w) : Error(kModelLoad, w) {} };
// The tensors of a folder do not fit the model; the text lists everything that is wrong.
struct QE_API WeightError : Error {
    std::vector<std::string> missing, unexpected, wrong_shape, wrong_type;
    explicit WeightError(const std::string& w) : Error(kModelLoad, w) {}
};
// A batch that cannot be run: unknown token id, position past the limit, request twice in a batch.
struct QE_API StepError : Error { explicit StepError(const std::string& w) : Error(kInvalidArg, w) {} };
// The pool has fewer free pages than were asked for.  Nothing was taken.
struct QE_API OutOfPages : Error { explicit OutOfPages(const std::string& w) : Error(kContextFull, w) {} };
// Every per-request state slot is in use.
struct QE_API OutOfSlots : Error { explicit OutOfSlots(const std::string& w) : Error(kKvCache, w) {} };
// A kernel launcher refused its arguments, a launch failed, a kernel gave up on a wait, or a library is missing.
struct QE_API KernelError : Error { explicit KernelError(const std::string& w) : Error(kKernelLaunch, w) {} };
// The bookkeeping found itself inconsistent (a page lost, held twice, freed twice).
struct QE_API CheckError : Error { explicit CheckError(const std::string& w) : Error(kInvalidState, w) {} };

// ---- element types ----------------------------------------------------------------------------------------
// F32 and BF16 carry the codes the kernel launchers take (PH_F32, PH_BF16).
enum class DType : int { F32 = 0, BF16 = 1, I32 = 2, F16 = 3, F64 = 4, I64 = 5, I16 = 6, I8 = 7, U8 = 8, BOOL = 9 };

inline size_t dtype_size(DType d) {
    switch (d) {
        case DType::F64: case DType::I64: return 8;
        case DType::F32: case DType::I32: return 4;
        case DType::BF16: case DType::F16: case DType::I16: return 2;
        default: return 1;
    }
}
inline const char* dtype_name(DType d) {
    switch (d) {
        case DType::F32: return "float32"; case DType::BF16: return "bfloat16"; case DType::I32: return "int32";
        case DType::F16: return "float16"; case DType::F64: return "float64"; case DType::I64: return "int64";
        case DType::I16: return "int16"; case DType::I8: return "int8"; case DType::U8: return "uint8";
        default: return "bool";
    }
}
inline bool dtype_is_float(DType d) { return d == DType::F32 || d == DType::BF16 || d == DType::F16 || d == DType::F64; }
inline bool dtype_is_int(DType d) { return d == DType::I32 || d == DType::I64 || d == DType::I16 || d == DType::I8 || d == DType::U8; }

// "bfloat16" / "bf16" / "float32" / "fp32": the two compute precisions.
inline DType parse_compute_dtype(const std::string& s) {
    if (s == "bfloat16" || s == "bf16") return DType::BF16;
    if (s == "float32" || s == "fp32") return DType::F32;
    throw Error(kInvalidArg, "dtype '" + s + "' is not supported (bfloat16 or float32)");
}

// ---- tensor view ------------------------------------------------------------------------------------------
struct Tensor {
    void* data = nullptr;
    DType dtype = DType::F32;
    std::vector<int64_t> shape;

    Tensor() = default;
    Tensor(void* p, DType d, std::vector<int64_t> s) : data(p), dtype(d), shape(std::move(s)) {}
    bool defined() const { return data != nullptr; }
    int64_t numel() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
    size_t bytes() const { return (size_t)numel() * dtype_size(dtype); }
    int64_t dim(int i) const { return shape.at(i < 0 ? shape.size() + i : i); }
    template <typename T> T* as() const { return static_cast<T*>(data); }
    int code() const { return (int)dtype; }         // for the kernel launchers: 0 float32, 1 bfloat16
    // rows [first, first + n) of a matrix or of a stack of matrices (along the first axis)
    Tensor rows(int64_t first, int64_t n) const {
        int64_t inner = 1;
        for (size_t i = 1; i < shape.size(); i++) inner *= shape[i];
        Tensor t(static_cast<char*>(data) + (size_t)(first * inner) * dtype_size(dtype), dtype, shape);
        t.shape[0] = n;
        return t;
    }
    Tensor view(std::vector<int64_t> s) const { return Tensor(data, dtype, std::move(s)); }
};

inline std::string shape_text(const std::vector<int64_t>& s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); i++) t += (i ? ", " : "") + std::to_string(s[i]);
    return t + "]";
}

// bfloat16 <-> float32 on the host (round to nearest even; NaN stays NaN).
inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

}  // namespace qe

// Device memory, scratch space and the kernel libraries, as the host library sees them.
//
// All device memory is plain cudaMalloc memory owned by a DeviceBuffer; a Workspace hands out named scratch
// tensors that keep their address from step to step (what a captured CUDA graph needs).  The kernels live in
// separate shared objects (libpurhie_core.so, libpurhie_flash.so, libpurhie_gemm100.so) that are opened by
// need from the folder this library was loaded from: a float32 model never touches the tensor-core libraries.
// A missing library is an error that says how to build it; there is no other implementation to fall back to.
#pragma once

#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.h"

namespace qe {

#define QE_CUDA(expr)                                                                                  \
    do {                                                                                               \
        cudaError_t qe_e_ = (expr);                                                                    \
        if (qe_e_ != cudaSuccess)                                                                      \
            throw ::qe::Error(qe_e_ == cudaErrorMemoryAllocation ? ::qe::kOutOfMemory : ::qe::kKernelLaunch, \
                              std::string(#expr) + ": " + cudaGetErrorString(qe_e_));                 \
    } while (0)

// Owns one cudaMalloc allocation.
class QE_API DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes);
    ~DeviceBuffer();
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    void* data() const { return p_; }
    size_t bytes() const { return n_; }
    void reset();
private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// Page-locked host memory.
class QE_API PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(size_t bytes);
    ~PinnedBuffer();
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    void* data() const { return p_; }
    size_t bytes() const { return n_; }
    void ensure(size_t bytes);          // grows (contents are lost)
private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// Device tensors that somebody keeps for good (weights and what parts derive from them).
class QE_API DeviceArena {
public:
    Tensor alloc(DType dtype, std::vector<int64_t> shape);
    void release(const Tensor& t);      // give one allocation back early (a temporary made while binding)
    size_t bytes() const { return bytes_; }
private:
    std::map<void*, DeviceBuffer> bufs_;
    size_t bytes_ = 0;
};

// Scratch tensors by name, reused from step to step and grown on demand.  A tensor of a given name keeps its
// address as long as requests do not outgrow it; `frozen` turns growth into an error (a captured graph points
// at these addresses).
class QE_API Workspace {
public:
    Workspace() = default;
    Tensor get(const std::string& name, std::vector<int64_t> shape, DType dtype);
    size_t bytes() const;
    bool frozen = false;
    cudaStream_t stream = nullptr;      // growing waits for this stream before the old block is freed
private:
    std::map<std::string, DeviceBuffer> bufs_;
};

// ---- kernel libraries ---------------------------------------------------------------------------------------
// Launcher prototypes (see the .cu files under csrc/).  Every launcher returns 0 or a status with a text.
struct CoreKernels {
    int (*embed_gather)(const void*, int, const int32_t*, float*, int, int, int, cudaStream_t);
    int (*add_rmsnorm)(float*, const void*, int, int, long long, const float*, float, const int32_t*, int, int, void*, int,
                       int, cudaStream_t);
    int (*swiglu)(const void*, int, int, long long, void*, int, int, int, cudaStream_t);
    int (*cast)(const void*, int, void*, int, long long, cudaStream_t);
    int (*qk_norm_rope_kv_write)(const void*, int, int, long long, const float*, const float*, const float*, float,
                                 const float*, int, int, const int32_t*, const int32_t*, void*, int, void*, void*, int,
                                 long long, int, int, int, int, int, int, const float*, int, int, float, cudaStream_t);
    int (*add_weight_sumsq)(float*, const void*, int, int, long long, const float*, int, int, void*, int, float*, int, cudaStream_t);
    int (*attention_generic)(const void*, int, const void*, const void*, int, long long, int, const int32_t*, int,
                             const int32_t*, const int32_t*, void*, int, int, int, int, int, int, float, cudaStream_t);
    int (*gemm_simple)(const void*, int, const void*, int, void*, int, int, int, int, cudaStream_t);
    int (*argmax)(const float*, int, int, int32_t*, void*, long long, cudaStream_t);   // several CTAs per row, with scratch
    long long (*argmax_scratch_bytes)(int);
    int (*sample_temperature)(const float*, int, int, const float*, const double*, float, int32_t*, cudaStream_t);
    int (*sample_chain)(const float*, int, int, const void*, int32_t*, cudaStream_t);
    int (*sample_chain_max_k)(void);
    int (*random_fill)(void*, int, long long, unsigned long long, int, double, double, cudaStream_t);
    const char* (*last_error)(void);
};
struct FlashKernels {
    int (*prefill)(const void*, const void*, const void*, long long, int, const int32_t*, int, const int32_t*,
                   const int32_t*, const int32_t*, const int32_t*, int, void*, int, int, int, int, float, cudaStream_t);
    int (*decode)(const void*, const void*, const void*, long long, int, const int32_t*, int, const int32_t*, int,
                  const int32_t*, const int32_t*, float*, float*, void*, int, int, int, int, int, float, cudaStream_t);
    int (*decode_bulk)(const void*, const void*, const void*, long long, int, int, const int32_t*, int, const int32_t*, int,
                       const int32_t*, const int32_t*, float*, float*, void*, int, int, int, int, int, float, int, int*,
                       cudaStream_t);
    int (*prefill_tc5)(const void*, int, const void*, const void*, long long, int, int, const int32_t*, int, const int32_t*,
                       const int32_t*, const int32_t*, const int32_t*, int, void*, int, int, int, int, float, int, float*,
                       float*, int*, cudaStream_t);
    const char* (*last_error)(void);
};
struct GemmKernels {
    int (*gemm)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int, const float*, int, int, float,
                const float*, void*, float*, int*, cudaStream_t);
    int (*gemm_pair)(const void*, const void*, void*, int, int, int, int, int, int, int, int, const float*, int, int, float,
                     const float*, void*, float*, int*, cudaStream_t);
    const char* (*last_error)(void);
};

// Folder the kernel libraries are opened from: set_library_dir(), else $PURHIE_B200_LIB_DIR, else the folder
// this library itself was loaded from.
QE_API void set_library_dir(const std::string& dir);
QE_API std::string library_dir();
QE_API const CoreKernels& core_kernels();
QE_API const FlashKernels& flash_kernels();
QE_API const GemmKernels& gemm_kernels();
QE_API void require_library(const std::string& name);      // "core", "flash", "gemm100": open it now
QE_API extern long long g_launches;                          // launcher calls so far (for the bench's count)

// Time per kernel class, for finding out where a step's time goes (the reference prints such a breakdown under
// QWEN_PROFILE=1: src/qwen_model.cpp:393-423, 2795-2818).  Off unless PURHIE_PROFILE=1 is in the environment (or
// set_enabled): then every launcher call is bracketed by CUDA events on the engine's stream, batches of single
// tokens are launched kernel by kernel instead of replayed as graphs, and report() gives, per launcher name, the
// calls, the device milliseconds and, where the caller noted them, the bytes and flops of its launches.  The
// events serialise nothing, but a profiled step is a little slower than an unprofiled one.
class QE_API LaunchProfile {
public:
    static LaunchProfile& get();
    bool on() const { return enabled_; }
    void set_enabled(bool on) { enabled_ = on; }
    void set_stream(cudaStream_t s) { stream_ = s; }
    void forget_stream(cudaStream_t s) { if (stream_ == s) stream_ = nullptr; }      // before s is destroyed
    void note_cost(double bytes, double flops) { pending_bytes_ = bytes; pending_flops_ = flops; }   // of the next launch
    void begin(const char* call_text);
    void end();
    // {"name": {"calls", "ms", "bytes", "flops"}} over everything since the last reset; waits for the stream.
    std::string report_json(bool reset);
    // Timing by omission: launchers named here (comma separated, "" for none) are not run from now on, so that a
    // graph captured afterwards shows what the rest costs without them.  The step's results are then meaningless.
    void leave_out(const char* names);
    bool leaves_out(const char* call_text) const { return !left_out_.empty() && is_left_out(call_text); }
private:
    bool is_left_out(const char* call_text) const;
    std::vector<std::string> left_out_;
    static std::string launcher_name(const char* call_text);
    LaunchProfile();
    struct Record { std::string name; cudaEvent_t start, stop; double bytes, flops; };
    bool enabled_ = false;
    cudaStream_t stream_ = nullptr;
    double pending_bytes_ = 0, pending_flops_ = 0;
    std::vector<Record> records_;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> spare_;
    struct Sum { long long calls = 0; double ms = 0, bytes = 0, flops = 0; };
    std::map<std::string, Sum> sums_;
    void fold();
};
struct LaunchScope {
    bool on;
    explicit LaunchScope(const char* call_text) : on(LaunchProfile::get().on()) { if (on) LaunchProfile::get().begin(call_text); }
    ~LaunchScope() { if (on) LaunchProfile::get().end(); }
};

// Run a launcher; a non-zero status becomes a KernelError with the library's text.
#define QE_LAUNCH(lib, call)                                                                     \
    do {                                                                                         \
        ::qe::g_launches++;                                                                      \
        ::qe::LaunchScope qe_scope_(#call);                                                      \
        if (::qe::LaunchProfile::get().leaves_out(#call)) break;                                 \
        if ((call) != 0) throw ::qe::KernelError((lib).last_error());                           \
    } while (0)

QE_API int sm_count();                                      // of the current device

}  // namespace qe

// Shared helpers of the kernel libraries: status codes, the thread-local error text, dtype codes and
// small device functions.  Every exported launcher returns PH_OK or sets the error text and returns a
// non-zero status; nothing here traps or spins without a bound.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <utility>

#define PH_OK 0
#define PH_ERR_ARG 1
#define PH_ERR_LAUNCH 2
#define PH_ERR_UNSUPPORTED 3

#define PH_F32 0
#define PH_BF16 1

// A library that compiles another library's source into itself defines PH_EXPORT first (hidden) to keep that
// source's entry points to itself.
#ifndef PH_EXPORT
#define PH_EXPORT extern "C" __attribute__((visibility("default")))
#endif

namespace ph {

inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PH_ERR_LAUNCH, "%s: launch failed: %s", what, cudaGetErrorString(e));
    return PH_OK;
}

inline bool valid_dtype(int d) { return d == PH_F32 || d == PH_BF16; }

// Programmatic dependent launch.  A kernel launched through launch_overlapped may start while the kernel
// before it in the stream is still running: its blocks become resident as soon as every block of that kernel has
// called pdl_launch_dependents() (or exited), run whatever does not depend on that kernel's results (set-up,
// prefetch of weights), and stop at pdl_wait() until that kernel has completed and its writes are visible.  Every
// such kernel calls pdl_wait() before it reads anything a predecessor produced and before it writes global
// memory at all.  PURHIE_PDL=0 in the environment turns the attribute off (the device calls are then no-ops).
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("PURHIE_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every thread gets the result.  The
// order of additions depends on NT only.
template <int NT> __device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < NT / 32) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

}  // namespace ph

// Dispatch on a dtype code: runs BODY with type alias NAME bound to float or __nv_bfloat16.
#define PH_DISPATCH(CODE, NAME, ...)                                  \
    do {                                                              \
        if ((CODE) == PH_F32) { using NAME = float; __VA_ARGS__; }    \
        else { using NAME = __nv_bfloat16; __VA_ARGS__; }             \
    } while (0)

// Every library exports its own copy of this under the library's prefix.
#define PH_DEFINE_LAST_ERROR(PREFIX) \
    PH_EXPORT const char* PREFIX##_last_error() { return ph::error_buffer(); }

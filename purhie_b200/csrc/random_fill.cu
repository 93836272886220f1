// Seeded random fill on the device: element i of the output is random_value(key, i), the very function the
// host uses when it writes a model folder (weights/random.h), so a model filled here has the bits of the same
// model written to a file and loaded.  One thread per element, grid-stride.
#include "common.cuh"
#include "../weights/random.h"

namespace {

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, unsigned long long key, int kind, double a, double b) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = ph::from_float<T>(qe::rnd::random_value(key, (unsigned long long)i, kind, a, b));
}

}  // namespace

// out[i] = N(0, a) (kind 0), U(a, b) (kind 1) or a (kind 2), rounded to out_dtype, for i < n.
PH_EXPORT int ph_random_fill(void* out, int out_dtype, long long n, unsigned long long key, int kind, double a, double b,
                             cudaStream_t stream) {
    if (!ph::valid_dtype(out_dtype)) return ph::fail(PH_ERR_ARG, "random_fill: out_dtype must be float32 or bfloat16");
    if (n < 0 || kind < 0 || kind > 2) return ph::fail(PH_ERR_ARG, "random_fill: bad size or kind");
    if (n == 0) return PH_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    PH_DISPATCH(out_dtype, T, random_fill_kernel<T><<<blocks, threads, 0, stream>>>((T*)out, n, key, kind, a, b));
    return ph::check_launch("random_fill");
}

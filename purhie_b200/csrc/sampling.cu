// Sampling on the device: greedy (argmax, lowest id wins ties) and temperature sampling.
//
// Temperature sampling follows the reference's chain with top-k, top-p and min-p switched off
// (src/sampler.cpp:120-127, 155-169): candidates are the tokens with logit >= max - 40, each weighs
// exp((logit - max) / T), and the token is the first one, in id order, whose running sum exceeds
// r * total, r being one uniform number in [0, 1) that the host draws per token.  Sums are in double.
// Greedy: src/sampler.cpp:60-68.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

constexpr int NT = 1024;

__global__ void __launch_bounds__(NT) argmax_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ out) {
    __shared__ float bv[NT / 32];
    __shared__ int bi[NT / 32];
    const float* row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += NT) {
        const float v = row[i];
        if (idx == 0x7fffffff || v > best) { best = v; idx = i; }   // i ascends: a tie keeps the lower id
    }
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = bv[lane];
        idx = bi[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
    }
}

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double t = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

__global__ void __launch_bounds__(NT) sample_temperature_kernel(const float* __restrict__ logits, int V,
                                                                const float* __restrict__ temperature,
                                                                const double* __restrict__ uniform, float range,
                                                                int32_t* __restrict__ out) {
    __shared__ double dscratch[32];
    __shared__ float fscratch[32];
    __shared__ double chunk_sum[NT];
    const float* row = logits + (size_t)blockIdx.x * V;
    const float T = temperature[blockIdx.x];
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += NT) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) fscratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = warp_max(fscratch[threadIdx.x & 31]);
    const float floor_logit = mx - range;
    // each thread owns a contiguous run of ids, so that a prefix over threads is a prefix over ids
    const int per = (V + NT - 1) / NT;
    const int lo = threadIdx.x * per, hi = min(V, lo + per);
    double mine = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v >= floor_logit) mine += (double)(float)exp((double)(v - mx) / (double)T);
    }
    chunk_sum[threadIdx.x] = mine;
    const double total = block_sum_double(mine, dscratch);
    const double r = uniform[blockIdx.x] * total;
    if (threadIdx.x == 0) {
        // walk the per-thread sums, then the ids inside the run that holds r
        double cum = 0.0;
        int pick = -1;
        for (int t = 0; t < NT && pick < 0; ++t) {
            const int tlo = t * per, thi = min(V, tlo + per);
            if (tlo >= thi) break;
            if (r < cum + chunk_sum[t]) {
                double c = cum;
                for (int i = tlo; i < thi; ++i) {
                    const float v = row[i];
                    if (v < floor_logit) continue;
                    c += (double)(float)exp((double)(v - mx) / (double)T);
                    if (r < c) { pick = i; break; }
                }
                cum = c;                       // rounding may put r just past this run: go on
            } else {
                cum += chunk_sum[t];
            }
        }
        if (pick < 0) {                        // r == total after rounding: the last candidate
            for (int i = V - 1; i >= 0; --i)
                if (row[i] >= floor_logit) { pick = i; break; }
        }
        out[blockIdx.x] = pick < 0 ? 0 : pick;
    }
}

}  // namespace

PH_EXPORT int ph_argmax(const float* logits, int R, int V, int32_t* out, cudaStream_t stream) {
    if (!logits || !out || R < 0 || V < 1) return fail(PH_ERR_ARG, "argmax: bad arguments (rows %d, V %d)", R, V);
    if (R == 0) return PH_OK;
    argmax_kernel<<<R, NT, 0, stream>>>(logits, V, out);
    return check_launch("argmax");
}

PH_EXPORT int ph_sample_temperature(const float* logits, int R, int V, const float* temperature,
                                    const double* uniform, float range, int32_t* out, cudaStream_t stream) {
    if (!logits || !out || !temperature || !uniform || R < 0 || V < 1 || !(range > 0.0f))
        return fail(PH_ERR_ARG, "sample_temperature: bad arguments (rows %d, V %d)", R, V);
    if (R == 0) return PH_OK;
    sample_temperature_kernel<<<R, NT, 0, stream>>>(logits, V, temperature, uniform, range, out);
    return check_launch("sample_temperature");
}

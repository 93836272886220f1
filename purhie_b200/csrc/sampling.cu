// Sampling on the device: greedy (argmax, lowest id wins ties) and temperature sampling.
//
// Temperature sampling follows the reference's chain with top-k, top-p and min-p switched off
// (src/sampler.cpp:120-127, 155-169): candidates are the tokens with logit >= max - 40, each weighs
// exp((logit - max) / T), and the token is the first one, in id order, whose running sum exceeds
// r * total, r being one uniform number in [0, 1) that the host draws per token.  Sums are in double.
// Greedy: src/sampler.cpp:60-68.
//
// The chain with top-k on (src/sampler.cpp:72-92, 127-169): one CTA per row finds the k best tokens (by logit
// descending, id ascending) with a radix selection over the order-preserving bits of the logits, sorts them, and
// one thread then walks the reference's loops as they stand: top-p over the candidates, min-p, temperature and the
// draw, in double where the reference uses double, with the uniform number the host drew for the token.
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

constexpr int KMAX = 256;          // most candidates the chain kernel keeps

// Bits that order like the floats they come from (-0 counted as +0).
__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t b = __float_as_uint(f + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One per-row parameter record, as the host packs it.
struct ChainRow {
    double uniform;
    float top_p, log_min_p, temperature;     // log_min_p: -inf when min-p is off
    int top_k;
};

__global__ void __launch_bounds__(NT) sample_chain_kernel(const float* __restrict__ logits, int V,
                                                          const ChainRow* __restrict__ rows, int32_t* __restrict__ out) {
    __shared__ int hist[256];
    __shared__ uint32_t sel_prefix, sel_mask;
    __shared__ int sel_remaining, n_gt;
    __shared__ int scan[NT / 32];
    __shared__ uint32_t cand_key[KMAX];
    __shared__ int cand_id[KMAX], sorted_id[KMAX];
    const float* row = logits + (size_t)blockIdx.x * V;
    const ChainRow prm = rows[blockIdx.x];
    const int k = min(min(prm.top_k, V), KMAX);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { sel_prefix = 0; sel_mask = 0; sel_remaining = k; n_gt = 0; }
    // ---- the key of the k-th best: eight bits at a time, from the top ----
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += NT) hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sel_prefix, mask = sel_mask;
        for (int i0 = 0; i0 < V; i0 += NT) {
            const int i = i0 + threadIdx.x;
            const bool in = i < V;
            const uint32_t key = in ? order_key(row[i]) : 0u;
            const bool take = in && (key & mask) == prefix;
            const int bin = take ? (int)((key >> shift) & 255u) : -1;
            // lanes with the same bin add once
            const unsigned peers = __match_any_sync(0xffffffffu, bin);
            if (take && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int acc = 0, b = 255;
            for (; b > 0; --b) {
                if (acc + hist[b] >= sel_remaining) break;
                acc += hist[b];
            }
            sel_remaining -= acc;                      // how many to take from bin b (and, in the end, of the key itself)
            sel_prefix |= (uint32_t)b << shift;
            sel_mask |= 255u << shift;
        }
        __syncthreads();
    }
    const uint32_t kth = sel_prefix;
    const int n_equal = sel_remaining;                 // tokens with exactly the k-th key to keep: the lowest ids
    // ---- collect: everything above the k-th key, then the first n_equal with the key itself, in id order ----
    const int per = (V + NT - 1) / NT;
    const int lo = threadIdx.x * per, hi = min(V, lo + per);
    int my_equal = 0;
    for (int i = lo; i < hi; ++i) {
        const uint32_t key = order_key(row[i]);
        if (key > kth) {
            const int slot = atomicAdd(&n_gt, 1);
            cand_key[slot] = key;
            cand_id[slot] = i;
        } else if (key == kth) {
            ++my_equal;
        }
    }
    // exclusive scan of my_equal over the threads (threads own ascending runs of ids)
    int incl = my_equal;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) scan[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = scan[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        scan[lane] = w;                                // inclusive over warps
    }
    __syncthreads();
    int before = incl - my_equal + (warp > 0 ? scan[warp - 1] : 0);
    const int base = k - n_equal;                      // = number of keys above the k-th
    if (my_equal > 0 && before < n_equal) {
        for (int i = lo; i < hi && before < n_equal; ++i) {
            if (order_key(row[i]) == kth) {
                cand_key[base + before] = kth;
                cand_id[base + before] = i;
                ++before;
            }
        }
    }
    __syncthreads();
    // ---- sort the k candidates: key descending, id ascending ----
    if (threadIdx.x < k) {
        const uint32_t key = cand_key[threadIdx.x];
        const int id = cand_id[threadIdx.x];
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += (cand_key[j] > key || (cand_key[j] == key && cand_id[j] < id)) ? 1 : 0;
        sorted_id[rank] = id;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    // ---- the reference's loops over the sorted candidates ----
    auto logit_of = [&](int j) { return row[sorted_id[j]] + 0.0f; };
    int n = k;
    if (prm.top_p < 1.0f) {
        const float mx = logit_of(0);
        double z = 0.0;
        for (int j = 0; j < n; ++j) z += exp((double)logit_of(j) - (double)mx);
        double cum = 0.0;
        int keep = n;
        for (int j = 0; j < n; ++j) {
            cum += exp((double)logit_of(j) - (double)mx);
            if (cum >= (double)prm.top_p * z) { keep = j + 1; break; }
        }
        n = keep;
    }
    // min-p: the candidates are sorted, so the survivors are a prefix
    {
        const float cut = logit_of(0) + prm.log_min_p;
        int keep = 0;
        for (int j = 0; j < n; ++j)
            if (!(logit_of(j) < cut)) ++keep; else break;
        n = keep > 0 ? keep : 1;
    }
    const float mx = logit_of(0);
    double z = 0.0;
    for (int j = 0; j < n; ++j) z += (double)(float)exp((double)(logit_of(j) - mx) / (double)prm.temperature);
    const double r = prm.uniform * z;
    double cum = 0.0;
    int pick = sorted_id[n - 1];
    for (int j = 0; j < n; ++j) {
        cum += (double)(float)exp((double)(logit_of(j) - mx) / (double)prm.temperature);
        if (r < cum) { pick = sorted_id[j]; break; }
    }
    out[blockIdx.x] = pick;
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

// rows: R records {double uniform; float top_p, log_min_p, temperature; int top_k} (24 bytes each) on the device.
// top_k of 1 .. 256 per row; temperature > 0.
PH_EXPORT int ph_sample_chain(const float* logits, int R, int V, const void* rows, int32_t* out, cudaStream_t stream) {
    if (!logits || !out || !rows || R < 0 || V < 1) return fail(PH_ERR_ARG, "sample_chain: bad arguments (rows %d, V %d)", R, V);
    static_assert(sizeof(ChainRow) == 24, "the host packs 24-byte records");
    if (R == 0) return PH_OK;
    sample_chain_kernel<<<R, NT, 0, stream>>>(logits, V, (const ChainRow*)rows, out);
    return check_launch("sample_chain");
}

PH_EXPORT int ph_sample_chain_max_k(void) { return KMAX; }

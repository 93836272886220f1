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
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
    int done = 0;
    if ((((uintptr_t)row) & 15) == 0) {
        // four values per load, four loads in flight per thread: one CTA reads a row of 150,000 logits, and how many
        // bytes it has under way decides how long that takes
        const float4* row4 = (const float4*)row;
        const int n4 = V >> 2;
        auto take = [&](const float4& q, int i) {                      // ids ascend inside a vector: a tie keeps the lower id
            if (idx == 0x7fffffff || q.x > best) { best = q.x; idx = i; }
            if (q.y > best) { best = q.y; idx = i + 1; }
            if (q.z > best) { best = q.z; idx = i + 2; }
            if (q.w > best) { best = q.w; idx = i + 3; }
        };
        int i = threadIdx.x;
        for (; i + 3 * NT < n4; i += 4 * NT) {
            const float4 a = row4[i], b = row4[i + NT], c = row4[i + 2 * NT], d = row4[i + 3 * NT];
            take(a, 4 * i); take(b, 4 * (i + NT)); take(c, 4 * (i + 2 * NT)); take(d, 4 * (i + 3 * NT));
        }
        for (; i < n4; i += NT) take(row4[i], 4 * i);
        done = n4 << 2;
    }
    for (int i = done + threadIdx.x; i < V; i += NT) {
        const float v = row[i];
        if (idx == 0x7fffffff || better(v, i, best, idx)) { best = v; idx = i; }
    }
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

// The same over several CTAs per row: a row of 150,000 logits read by one SM takes as long as a small product, because
// one SM has only so many bytes under way.  CTA (row, part) finds the best of its part of the row; the CTA that
// arrives last at the row's counter (no waiting: the others have left by then) picks among the parts in ascending
// order, so that a tie still goes to the lowest id, and puts the counter back to zero for the next call.
constexpr int PARTS_THREADS = 256;
constexpr int MAX_PARTS = 64;

__global__ void __launch_bounds__(PARTS_THREADS)
argmax_parts_kernel(const float* __restrict__ logits, int V, int per_part, int32_t* __restrict__ out, int* __restrict__ counters,
                    float* __restrict__ part_val, int* __restrict__ part_idx) {
    __shared__ float bv[PARTS_THREADS / 32];
    __shared__ int bi[PARTS_THREADS / 32];
    __shared__ int last;
    const int r = blockIdx.x, c = blockIdx.y, parts = gridDim.y;
    const float* row = logits + (size_t)r * V;
    const int lo = c * per_part, hi = min(V, lo + per_part);
    auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
    float best = -INFINITY;
    int idx = 0x7fffffff;
    int done = lo;
    if ((((uintptr_t)(row + lo)) & 15) == 0 && hi > lo) {
        const float4* p4 = (const float4*)(row + lo);
        const int n4 = (hi - lo) >> 2;
        auto take = [&](const float4& q, int i) {                      // ids ascend inside a vector: a tie keeps the lower id
            const int id = lo + 4 * i;
            if (idx == 0x7fffffff || q.x > best) { best = q.x; idx = id; }
            if (q.y > best) { best = q.y; idx = id + 1; }
            if (q.z > best) { best = q.z; idx = id + 2; }
            if (q.w > best) { best = q.w; idx = id + 3; }
        };
        int i = threadIdx.x;
        for (; i + 3 * PARTS_THREADS < n4; i += 4 * PARTS_THREADS) {    // four loads under way per thread
            const float4 a = p4[i], b = p4[i + PARTS_THREADS], c4 = p4[i + 2 * PARTS_THREADS], d = p4[i + 3 * PARTS_THREADS];
            take(a, i); take(b, i + PARTS_THREADS); take(c4, i + 2 * PARTS_THREADS); take(d, i + 3 * PARTS_THREADS);
        }
        for (; i < n4; i += PARTS_THREADS) take(p4[i], i);
        done = lo + (n4 << 2);
    }
    for (int i = done + threadIdx.x; i < hi; i += PARTS_THREADS) {
        const float v = row[i];
        if (idx == 0x7fffffff || better(v, i, best, idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < PARTS_THREADS / 32; ++w)
            if (better(bv[w], bi[w], best, idx)) { best = bv[w]; idx = bi[w]; }
        part_val[(size_t)r * parts + c] = best;
        part_idx[(size_t)r * parts + c] = idx;
        __threadfence();                                            // the part is visible before the arrival is
        last = atomicAdd(&counters[r], 1) == parts - 1;
    }
    __syncthreads();
    if (!last || warp != 0) return;
    __threadfence();
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int k = lane; k < parts; k += 32) {
        const float v = __ldcg(&part_val[(size_t)r * parts + k]);
        const int i = __ldcg(&part_idx[(size_t)r * parts + k]);
        if (better(v, i, best, idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if (lane == 0) {
        out[r] = idx == 0x7fffffff ? 0 : idx;
        counters[r] = 0;
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

constexpr int LIST_MAX = 6144;     // most tokens the chain kernel compacts into shared memory before it selects
constexpr int CHAIN_SMEM = LIST_MAX * 8;

// Inclusive scan of v over the block's threads in thread order; scratch holds one int per warp.
__device__ __forceinline__ int block_scan_inclusive(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = scratch[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        scratch[lane] = w;
    }
    __syncthreads();
    return incl + (warp > 0 ? scratch[warp - 1] : 0);
}

// Warp 0, all lanes: the bin of hist (walking down from 255) in which the remaining-th largest lies; returns the bin
// and, through taken, how many lie in the bins above it.
__device__ __forceinline__ int pick_bin(const int* hist, int remaining, int& taken) {
    const int lane = threadIdx.x & 31;
    // lane l owns bins 255 - 8 l .. 248 - 8 l, so that lanes ascend as bins descend
    int c[8], mine = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { c[j] = hist[255 - 8 * lane - j]; mine += c[j]; }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    const unsigned reach = __ballot_sync(0xffffffffu, incl >= remaining);
    const int owner = reach ? __ffs(reach) - 1 : 31;
    int bin = 0, above = 0;
    if (lane == owner) {
        int acc = incl - mine;
        int j = 0;
        for (; j < 7; ++j) {
            if (acc + c[j] >= remaining) break;
            acc += c[j];
        }
        bin = 255 - 8 * lane - j;
        above = acc;
    }
    bin = __shfl_sync(0xffffffffu, bin, owner);
    taken = __shfl_sync(0xffffffffu, above, owner);
    return bin;
}

// Radix selection, eight bits a pass from the top, of the rank-th largest of the values the callback yields for
// items 0 .. n-1 (it returns false for items that do not take part).  Returns the value; rank becomes how many items
// with exactly that value are still to be taken.  All threads call it.
template <typename Get>
__device__ __forceinline__ uint32_t radix_select(int n, int& rank, int* hist, uint32_t* sel, Get get) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { sel[0] = 0; sel[1] = 0; sel[2] = (uint32_t)rank; }
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += NT) hist[i] = 0;
        __syncthreads();
        const uint32_t prefix = sel[0], mask = sel[1];
        for (int i0 = 0; i0 < n; i0 += NT) {
            const int i = i0 + threadIdx.x;
            uint32_t key = 0;
            const bool take = i < n && get(i, key) && (key & mask) == prefix;
            const int bin = take ? (int)((key >> shift) & 255u) : -1;
            const unsigned peers = __match_any_sync(0xffffffffu, bin);          // lanes with the same bin add once
            if (take && lane == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
        }
        __syncthreads();
        if (warp == 0) {
            int taken;
            const int b = pick_bin(hist, (int)sel[2], taken);
            __syncwarp();
            if (lane == 0) { sel[2] -= (uint32_t)taken; sel[0] |= (uint32_t)b << shift; sel[1] |= 255u << shift; }
        }
        __syncthreads();
    }
    rank = (int)sel[2];
    return sel[0];
}

// The k best of a row (logit descending, id ascending) into cand_key / cand_id, in any order.
//
// A pass over the row finds the largest logit.  A second pass copies the tokens whose key shares the maximum's top
// eight bits (positive logits down to half the maximum, at the least) into a list in shared memory; if those are
// fewer than k the pass is repeated one bin further down, up to three times.  The k best are then selected in the
// list: by key, and among equal keys at the k-th place by id, lowest first.  A row for which no such list of k to
// LIST_MAX tokens exists (nearly flat, or spread over many powers of two) is selected from directly, with four
// passes over the row for the key and a walk in id order for the ties.
__device__ void select_top_k(const float* __restrict__ row, int V, int k, unsigned char* dyn, uint32_t* cand_key, int* cand_id) {
    __shared__ int hist[256];
    __shared__ int scratch[32];
    __shared__ float warp_max_v[32];
    __shared__ uint32_t sel[3];
    __shared__ int n_gt, n_list;
    uint32_t* list_key = (uint32_t*)dyn;                          // [LIST_MAX]
    int* list_id = (int*)(list_key + LIST_MAX);                   // [LIST_MAX]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int UNROLL = 8;                                     // loads in flight per thread
    if (threadIdx.x == 0) n_gt = 0;
    // ---- the largest logit ----
    float mx = -INFINITY;
    for (int i0 = 0; i0 < V; i0 += NT * UNROLL) {
        float v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int i = i0 + u * NT + threadIdx.x;
            v[u] = i < V ? row[i] : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) mx = fmaxf(mx, v[u]);
    }
    mx = warp_max(mx);
    if (lane == 0) warp_max_v[warp] = mx;
    __syncthreads();
    mx = warp_max(warp_max_v[lane]);
    const int b_max = (int)(order_key(mx) >> 24);
    // ---- the tokens near the maximum into the list ----
    bool listed = false;
    for (int j = 0; j < 4 && b_max - j >= 0 && !listed; ++j) {
        const uint32_t key_lo = (uint32_t)(b_max - j) << 24;      // the smallest key of the bin
        const float t = key_lo == 0 ? -INFINITY : __uint_as_float((key_lo & 0x80000000u) ? (key_lo & 0x7fffffffu) : ~key_lo);
        __syncthreads();
        if (threadIdx.x == 0) n_list = 0;
        __syncthreads();
        for (int i0 = 0; i0 < V; i0 += NT * UNROLL) {
            float v[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * NT + threadIdx.x;
                v[u] = i < V ? row[i] : -INFINITY;
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * NT + threadIdx.x;
                const bool take = i < V && v[u] >= t;
                const unsigned m = __ballot_sync(0xffffffffu, take);
                if (m) {                                           // rare: one shared counter, bumped once per warp
                    int base = 0;
                    if (lane == 0) base = atomicAdd(&n_list, __popc(m));
                    base = __shfl_sync(0xffffffffu, base, 0);
                    const int slot = base + __popc(m & ((1u << lane) - 1u));
                    if (take && slot < LIST_MAX) { list_key[slot] = order_key(v[u]); list_id[slot] = i; }
                }
            }
        }
        __syncthreads();
        if (n_list > LIST_MAX) break;                              // the bins further down hold more still
        listed = n_list >= k;
    }
    __syncthreads();
    if (listed) {
        const int n = n_list;
        int n_equal = k;
        const uint32_t kth = radix_select(n, n_equal, hist, sel, [&](int i, uint32_t& key) { key = list_key[i]; return true; });
        // how many share the k-th key; if more than are wanted, the wanted ones are those with the lowest ids
        int mine = 0;
        for (int i = threadIdx.x; i < n; i += NT) mine += list_key[i] == kth;
        if (threadIdx.x == 0) scratch[0] = 0;
        __syncthreads();
        if (mine) atomicAdd(&scratch[0], mine);
        __syncthreads();
        const int same = scratch[0];
        __syncthreads();
        uint32_t id_cut = 0xffffffffu;                             // ids up to this one are taken among the equal keys
        if (same > n_equal) {
            // the n_equal-th smallest id = the (same - n_equal + 1)-th largest
            int rank = same - n_equal + 1;
            id_cut = radix_select(n, rank, hist, sel, [&](int i, uint32_t& key) { key = (uint32_t)list_id[i]; return list_key[i] == kth; });
        }
        for (int i = threadIdx.x; i < n; i += NT) {
            const uint32_t key = list_key[i];
            if (key > kth || (key == kth && (uint32_t)list_id[i] <= id_cut)) {
                const int slot = atomicAdd(&n_gt, 1);
                cand_key[slot] = key;
                cand_id[slot] = list_id[i];
            }
        }
    } else {
        // ---- selection over the row itself ----
        int n_equal = k;
        const uint32_t kth = radix_select(V, n_equal, hist, sel, [&](int i, uint32_t& key) { key = order_key(row[i]); return true; });
        // threads own ascending runs of ids, so a prefix over threads is a prefix over ids
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
        int before = block_scan_inclusive(my_equal, scratch) - my_equal;
        const int base = k - n_equal;
        for (int i = lo; i < hi && my_equal > 0 && before < n_equal; ++i) {
            if (order_key(row[i]) == kth) {
                cand_key[base + before] = kth;
                cand_id[base + before] = i;
                ++before;
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(NT) sample_chain_kernel(const float* __restrict__ logits, int V,
                                                          const ChainRow* __restrict__ rows, int32_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ uint32_t cand_key[KMAX];
    __shared__ int cand_id[KMAX], sorted_id[KMAX];
    __shared__ float sorted_logit[KMAX];
    __shared__ double e_top_p[KMAX];
    __shared__ float e_draw[KMAX];
    const float* row = logits + (size_t)blockIdx.x * V;
    const ChainRow prm = rows[blockIdx.x];
    const int k = min(min(prm.top_k, V), KMAX);
    select_top_k(row, V, k, dyn, cand_key, cand_id);
    // ---- sort the k candidates: key descending, id ascending ----
    if (threadIdx.x < k) {
        const uint32_t key = cand_key[threadIdx.x];
        const int id = cand_id[threadIdx.x];
        int rank = 0;
        for (int j = 0; j < k; ++j) rank += (cand_key[j] > key || (cand_key[j] == key && cand_id[j] < id)) ? 1 : 0;
        sorted_id[rank] = id;
        sorted_logit[rank] = row[id] + 0.0f;
    }
    __syncthreads();
    // the exponentials of the reference's loops, one per thread; the sums stay with one thread, in its order
    if (threadIdx.x < k) {
        const float mx = sorted_logit[0];
        e_top_p[threadIdx.x] = exp((double)sorted_logit[threadIdx.x] - (double)mx);
        e_draw[threadIdx.x] = (float)exp((double)(sorted_logit[threadIdx.x] - mx) / (double)prm.temperature);
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    int n = k;
    if (prm.top_p < 1.0f) {
        double z = 0.0;
        for (int j = 0; j < n; ++j) z += e_top_p[j];
        double cum = 0.0;
        int keep = n;
        for (int j = 0; j < n; ++j) {
            cum += e_top_p[j];
            if (cum >= (double)prm.top_p * z) { keep = j + 1; break; }
        }
        n = keep;
    }
    {
        // min-p: the candidates are sorted, so the survivors are a prefix
        const float cut = sorted_logit[0] + prm.log_min_p;
        int keep = 0;
        for (int j = 0; j < n; ++j)
            if (!(sorted_logit[j] < cut)) ++keep; else break;
        n = keep > 0 ? keep : 1;
    }
    double z = 0.0;
    for (int j = 0; j < n; ++j) z += (double)e_draw[j];
    const double r = prm.uniform * z;
    double cum = 0.0;
    int pick = sorted_id[n - 1];
    for (int j = 0; j < n; ++j) {
        cum += (double)e_draw[j];
        if (r < cum) { pick = sorted_id[j]; break; }
    }
    out[blockIdx.x] = pick;
}

}  // namespace

// scratch: device memory of at least ph_argmax_scratch_bytes(R) bytes, zero before the first call (the kernel leaves
// its counters, the first 4 bytes per row the scratch has room for, at zero); calls that share a scratch must not
// overlap and must give its size the same way.
PH_EXPORT long long ph_argmax_scratch_bytes(int R) { return (long long)R * (4 + (long long)MAX_PARTS * 8); }

PH_EXPORT int ph_argmax_parts(const float* logits, int R, int V, int32_t* out, void* scratch, long long scratch_bytes,
                              cudaStream_t stream) {
    if (!logits || !out || R < 0 || V < 1) return fail(PH_ERR_ARG, "argmax: bad arguments (rows %d, V %d)", R, V);
    if (R == 0) return PH_OK;
    // parts of about 4,096 values, as many as fill the device once, a multiple of four values each
    int parts = (2 * 148 + R - 1) / R;
    parts = parts < 1 ? 1 : (parts > MAX_PARTS ? MAX_PARTS : parts);
    if (parts > (V + 4095) / 4096) parts = (V + 4095) / 4096;
    if (parts <= 1 || !scratch || scratch_bytes < ph_argmax_scratch_bytes(R) || R > 65535) {
        argmax_kernel<<<R, NT, 0, stream>>>(logits, V, out);
        return check_launch("argmax");
    }
    const int per_part = (((V + parts - 1) / parts) + 3) & ~3;
    // the counters keep their place whatever the number of rows of a call: they must be found at zero by the next one
    const long long rows_cap = scratch_bytes / (4 + (long long)MAX_PARTS * 8);
    int* counters = (int*)scratch;
    float* part_val = (float*)(counters + rows_cap);
    int* part_idx = (int*)(part_val + (size_t)rows_cap * MAX_PARTS);
    argmax_parts_kernel<<<dim3(R, parts), PARTS_THREADS, 0, stream>>>(logits, V, per_part, out, counters, part_val, part_idx);
    return check_launch("argmax");
}

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
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(sample_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CHAIN_SMEM) != cudaSuccess)
            return fail(PH_ERR_LAUNCH, "sample_chain: cannot reserve %d bytes of shared memory", CHAIN_SMEM);
        configured = true;
    }
    sample_chain_kernel<<<R, NT, CHAIN_SMEM, stream>>>(logits, V, (const ChainRow*)rows, out);
    return check_launch("sample_chain");
}

PH_EXPORT int ph_sample_chain_max_k(void) { return KMAX; }

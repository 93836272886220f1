// Attention over cache pages, the plain kernel: any head size, any number of heads and groups, float32
// arithmetic.  It is the whole attention of the 32-bit path, the reference the fast kernels are tested
// against, and the refuge for head sizes the fast kernels do not take.
//
// One warp per (token row, query head).  The row at absolute position z of a request sees the cached
// positions lo .. z, lo = max(0, z - window + 1) (window 0: lo = 0).  Keys are taken 32 at a time
// starting from lo: each lane scores one key (the whole dot product in one lane, in d order), the warp
// keeps a running maximum and sum (online softmax) and each lane owns the output dimensions d = lane,
// lane + 32, ...  The order of every addition depends on (z, window) only, never on how the request was
// cut into steps or on what else is in the batch.
// Formulas (reference): src/qwen_ops.cpp:26-51 (scores * scale, max-subtracted softmax, weighted sum of
// V; query head h uses kv head h / (HQ / HKV)); window: src/attention.h:73.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

constexpr int WARPS = 4;
constexpr int MAX_D = 512;

template <typename TQ, typename TKV, typename TO>
__global__ void attention_generic_kernel(const TQ* __restrict__ q, const TKV* __restrict__ k_base,
                                         const TKV* __restrict__ v_base, long long page_stride, int page_size,
                                         const int32_t* __restrict__ block_table, int table_stride,
                                         const int32_t* __restrict__ row_seg, const int32_t* __restrict__ positions,
                                         TO* __restrict__ out, int T, int HQ, int HKV, int D, int window, float scale) {
    __shared__ float qs[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)T * HQ) return;
    const int t = (int)(item / HQ), h = (int)(item % HQ);
    const int g = h / (HQ / HKV);
    const int z = positions[t];
    const int lo = (window > 0 && z - window + 1 > 0) ? z - window + 1 : 0;
    const int32_t* table = block_table + (size_t)row_seg[t] * table_stride;
    const TQ* qr = q + ((size_t)t * HQ + h) * D;
    for (int d = lane; d < D; d += 32) qs[warp][d] = to_float<TQ>(qr[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.0f;
    float acc[MAX_D / 32];
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.0f;

    for (int base = lo; base <= z; base += 32) {
        const int p = base + lane;
        float s = -INFINITY;
        const TKV* vrow = nullptr;
        if (p <= z) {
            const int page = table[p / page_size];
            const size_t off = (size_t)page * page_stride + ((size_t)g * page_size + p % page_size) * D;
            const TKV* krow = k_base + off;
            vrow = v_base + off;
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot += qs[warp][d] * to_float<TKV>(krow[d]);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pexp = (p <= z) ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);            // m = -inf on the first chunk: corr = 0, l and acc are 0
        l = l * corr + warp_sum(pexp);
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= corr;
        const int n = (z - base + 1) < 32 ? (z - base + 1) : 32;
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pexp, j);
            const unsigned long long vp = __shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
            const TKV* vj = (const TKV*)vp;
#pragma unroll
            for (int i = 0; i < MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] += pj * to_float<TKV>(vj[d]);
            }
        }
        m = m_new;
    }
    TO* o = out + ((size_t)t * HQ + h) * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) o[d] = from_float<TO>(acc[i] * inv);
    }
}

}  // namespace

PH_EXPORT int ph_attention_generic(const void* q, int q_dtype, const void* k_base, const void* v_base, int kv_dtype,
                                   long long page_stride, int page_size, const int32_t* block_table,
                                   int table_stride, const int32_t* row_seg, const int32_t* positions, void* out,
                                   int out_dtype, int T, int HQ, int HKV, int D, int window, float scale,
                                   cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !row_seg || !positions || !out || T < 0 || HQ < 1 || HKV < 1 ||
        D < 1 || page_size < 1 || window < 0 || !valid_dtype(q_dtype) || !valid_dtype(kv_dtype) ||
        !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "attention_generic: bad arguments (T %d, HQ %d, HKV %d, D %d)", T, HQ, HKV, D);
    if (HQ % HKV) return fail(PH_ERR_ARG, "attention_generic: %d query heads are not a multiple of %d kv heads", HQ, HKV);
    if (D > MAX_D) return fail(PH_ERR_UNSUPPORTED, "attention_generic: head_dim %d exceeds the supported %d", D, MAX_D);
    if (T == 0) return PH_OK;
    const long long items = (long long)T * HQ;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
#define LAUNCH(TQ, TKV, TO)                                                                                    \
    attention_generic_kernel<TQ, TKV, TO><<<blocks, WARPS * 32, 0, stream>>>(                                  \
        (const TQ*)q, (const TKV*)k_base, (const TKV*)v_base, page_stride, page_size, block_table, table_stride, \
        row_seg, positions, (TO*)out, T, HQ, HKV, D, window, scale)
    PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, PH_DISPATCH(out_dtype, TO, LAUNCH(TQ, TKV, TO))));
#undef LAUNCH
    return check_launch("attention_generic");
}

// Per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into cache pages,
// in one launch over the fused [q | k | v] rows that the projection produced.
//
// One warp per (token, head).  For a q or k head: optional bias, v = v * rsqrt(mean_D(v^2) + eps) * w,
// then rotate-half pairs (i, i + n_rot/2): (a, b) -> (a cos - b sin, a sin + b cos) with the angle of the
// token's absolute position (interleaved = 1 pairs (2i, 2i + 1) instead); dimensions >= n_rot pass
// through.  A v head is only biased and copied.  The table row of a position holds n_rot / 2 cosines, then
// n_rot / 2 sines, one per pair.
// Sums and angles are float32; the cos/sin table is made on the host in double precision.
// Reference: src/attention.hip:273-313 (attn_prep: bias, norm, rotation, cache write), :219-240
// (the norm and the rotation), src/qwen_ops.cpp:15-24 (rotate-half pairing).
//
// Cache addressing: token slot s = page * page_size + offset; element (s, head h, d) of K lives at
// k_base + page * page_stride + (h * page_size + offset) * D + d, and the same for V from v_base.
#include "common.cuh"

namespace {

using namespace ph;

constexpr int WARPS = 4;
constexpr int MAX_D = 512;

template <typename TI, typename TQ, typename TKV>
__global__ void qk_norm_rope_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                    const float* __restrict__ bias, const float* __restrict__ q_w,
                                    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                    int n_rot, int max_pos, const int32_t* __restrict__ positions,
                                    const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                    TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                    int page_size, int HQ, int HKV, int D, int interleaved) {
    __shared__ float buf[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * WARPS + warp;
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    if (head >= n_heads) return;
    const int width = n_heads * D;
    const TI* src = qkv + (size_t)t * width + (size_t)head * D;
    const float* b = bias ? bias + (size_t)head * D : nullptr;
    const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
    float* row = buf[warp];

    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) {
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += to_float<TI>(src[(size_t)s * split_stride + d]);
        if (b) v += b[d];
        row[d] = v;
        ss += v * v;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    if (!is_q && !is_k) {
        // v head: copy
        if (!slot_mapping) return;
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int h = head - HQ - HKV;
        TKV* dst = v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D;
        __syncwarp();
        for (int d = lane; d < D; d += 32) dst[d] = from_float<TKV>(row[d]);
        return;
    }
    if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) row[d] = row[d] * inv * w[d];
    }
    __syncwarp();
    float outv[MAX_D / 32];
    const int half = n_rot / 2;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);     // positions are validated on the host
    const float* cs = cos_sin ? cos_sin + (size_t)pos * n_rot : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d >= D) break;
        float v = row[d];
        if (cs && d < n_rot) {
            if (interleaved) {
                const int j = d >> 1;
                const float c = cs[j], s = cs[half + j];
                v = (d & 1) ? row[d - 1] * s + row[d] * c : row[d] * c - row[d + 1] * s;
            } else {
                const int j = d < half ? d : d - half;
                const float c = cs[j], s = cs[half + j];
                v = d < half ? row[d] * c - row[d + half] * s : row[d - half] * s + row[d] * c;
            }
        }
        outv[i] = v;
    }
    if (is_q) {
        TQ* dst = q_out + ((size_t)t * HQ + head) * D;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) break;
            dst[d] = from_float<TQ>(outv[i]);
        }
    } else if (slot_mapping) {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int h = head - HQ;
        TKV* dst = k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) break;
            dst[d] = from_float<TKV>(outv[i]);
        }
    }
}

}  // namespace

PH_EXPORT int ph_qk_norm_rope_kv_write(const void* qkv, int qkv_dtype, int splits, long long split_stride,
                                       const float* bias, const float* q_norm_w, const float* k_norm_w, float eps,
                                       const float* cos_sin, int n_rot, int max_pos, const int32_t* positions,
                                       const int32_t* slot_mapping, void* q_out, int q_dtype, void* k_base,
                                       void* v_base, int kv_dtype, long long page_stride, int page_size, int T,
                                       int HQ, int HKV, int D, int interleaved, cudaStream_t stream) {
    if (!qkv || !positions || !q_out || T < 0 || HQ < 1 || HKV < 0 || D < 2 || splits < 1 || !valid_dtype(qkv_dtype) ||
        !valid_dtype(q_dtype) || !valid_dtype(kv_dtype))
        return fail(PH_ERR_ARG, "qk_norm_rope: bad arguments (T %d, HQ %d, HKV %d, D %d)", T, HQ, HKV, D);
    if (D > MAX_D) return fail(PH_ERR_UNSUPPORTED, "qk_norm_rope: head_dim %d exceeds the supported %d", D, MAX_D);
    if (cos_sin && (n_rot < 2 || n_rot > D || (n_rot & 1) || max_pos < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: rotary width %d must be even and at most head_dim %d", n_rot, D);
    if (slot_mapping && (!k_base || !v_base || page_size < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: a cache write needs the pool and its page size");
    if (T == 0) return PH_OK;
    dim3 grid(T, (HQ + 2 * HKV + WARPS - 1) / WARPS);
#define LAUNCH(TI, TQ, TKV)                                                                                       \
    qk_norm_rope_kernel<TI, TQ, TKV><<<grid, WARPS * 32, 0, stream>>>(                                            \
        (const TI*)qkv, splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, n_rot, max_pos, positions,  \
        slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, D, interleaved)
    PH_DISPATCH(qkv_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH(TI, TQ, TKV))));
#undef LAUNCH
    return check_launch("qk_norm_rope");
}

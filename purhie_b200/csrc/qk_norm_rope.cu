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

// A factor per token that the norm in front of the qkv product left out: rsqrt(sum over the chunks of sumsq[t][chunk] /
// width + eps).  The product is linear, so the factor is applied to its result here (before the bias).  sumsq null: 1.
struct RowFactor {
    const float* sumsq;
    int chunks, width;
    float eps;
};
__device__ __forceinline__ float row_factor(const RowFactor& rf, int t) {
    if (!rf.sumsq) return 1.0f;
    float s = 0.0f;
    for (int k = 0; k < rf.chunks; ++k) s += rf.sumsq[(size_t)t * rf.chunks + k];
    return rsqrtf(s / (float)rf.width + rf.eps);
}
constexpr int MAX_D = 512;

template <typename TI, typename TQ, typename TKV>
__global__ void qk_norm_rope_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                    const float* __restrict__ bias, const float* __restrict__ q_w,
                                    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                    int n_rot, int max_pos, const int32_t* __restrict__ positions,
                                    const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                    TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                    int page_size, int HQ, int HKV, int D, int interleaved, RowFactor rf) {
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
    const float rs = row_factor(rf, t);

    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) {
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += to_float<TI>(src[(size_t)s * split_stride + d]);
        v *= rs;
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

// Fast path for head_dim 128 rotated over its whole width in half pairs, for a few tokens (where the launch is
// short of warps): one warp per token and HPW consecutive heads (1 as launched),
// four consecutive dimensions per lane, every load in flight at once, the rotation partner (64 dimensions away)
// fetched from lane ^ 16 by shuffle.  The order of the additions is the same for every launch shape.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TI, typename TQ, typename TKV, int HPW>
__global__ void qk_norm_rope_d128_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                         const float* __restrict__ bias, const float* __restrict__ q_w,
                                         const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                         int max_pos, const int32_t* __restrict__ positions,
                                         const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                         TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                         int page_size, int HQ, int HKV, RowFactor rf) {
    constexpr int D = 128;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = (blockIdx.y * WARPS + warp) * HPW;      // this warp's HPW consecutive heads of token t
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    if (head0 >= n_heads) return;
    const int d0 = lane * 4;
    // what no kernel of this step writes (positions, slots, the table, the norms' weights) is fetched while the
    // kernel in front still runs
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float4 c = make_float4(1.0f, 1.0f, 1.0f, 1.0f), sn = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (cos_sin) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        const int j = (lane & 15) * 4;                       // pair index of this lane's first dimension
        c = ld4(cos_sin + (size_t)pos * D + j);
        sn = ld4(cos_sin + (size_t)pos * D + 64 + j);
    }
    const float4 gq = q_w ? ld4(q_w + d0) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    const float4 gk = k_w ? ld4(k_w + d0) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    pdl_wait();
    const float rs = row_factor(rf, t);
    // every head's loads are issued before any of them is used
    float4 v[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (head0 + i >= n_heads) continue;
        const TI* src = qkv + (size_t)t * n_heads * D + (size_t)(head0 + i) * D + d0;
        for (int s0 = 0; s0 < splits; s0 += 8) {             // eight partial sums in flight, added in order
            float4 u[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                u[j] = s0 + j < splits ? ld4(src + (size_t)(s0 + j) * split_stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) { v[i].x += u[j].x; v[i].y += u[j].y; v[i].z += u[j].z; v[i].w += u[j].w; }
        }
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int head = head0 + i;
        if (head >= n_heads) break;
        float4 x = make_float4(v[i].x * rs, v[i].y * rs, v[i].z * rs, v[i].w * rs);
        if (bias) {
            const float4 b = ld4(bias + (size_t)head * D + d0);
            x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
        }
        const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
        if (!is_q && !is_k) {
            if (slot < 0) continue;
            const int h = head - HQ - HKV;
            st4(v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
            continue;
        }
        const float* w = is_q ? q_w : k_w;
        if (w) {
            const float ss = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
            const float inv = rsqrtf(ss / (float)D + eps);
            const float4 g = is_q ? gq : gk;
            x.x = x.x * inv * g.x; x.y = x.y * inv * g.y; x.z = x.z * inv * g.z; x.w = x.w * inv * g.w;
        }
        if (cos_sin) {
            float4 o;
            o.x = __shfl_xor_sync(0xffffffffu, x.x, 16); o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
            o.z = __shfl_xor_sync(0xffffffffu, x.z, 16); o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
            if (lane < 16) {       // first half: a cos - b sin
                x.x = x.x * c.x - o.x * sn.x; x.y = x.y * c.y - o.y * sn.y; x.z = x.z * c.z - o.z * sn.z; x.w = x.w * c.w - o.w * sn.w;
            } else {               // second half: a sin + b cos (a is the partner)
                x.x = o.x * sn.x + x.x * c.x; x.y = o.y * sn.y + x.y * c.y; x.z = o.z * sn.z + x.z * c.z; x.w = o.w * sn.w + x.w * c.w;
            }
        }
        if (is_q) {
            st4(q_out + ((size_t)t * HQ + head) * D + d0, x);
        } else if (slot >= 0) {
            const int h = head - HQ;
            st4(k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
        }
    }
}

// The same for many tokens: eight consecutive dimensions per lane (one 16-byte load of bfloat16), a half-warp per
// head, a warp walks ITERS pairs of heads of one token with every load issued first.  The sum of squares is added
// in the order of the kernel above (four-element groups, then a butterfly over the 32 groups: here over 16 lanes
// for the even and the odd group apart, then the two), so both give the same bits.  The rotation partner (64
// dimensions away) sits eight lanes away in the same half-warp.
struct F8 { float4 a, b; };
__device__ __forceinline__ F8 ld8(const float* p) { return {ld4(p), ld4(p + 4)}; }
__device__ __forceinline__ F8 ld8(const __nv_bfloat16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    return {make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1])),
            make_float4(__low2float(h[2]), __high2float(h[2]), __low2float(h[3]), __high2float(h[3]))};
}
__device__ __forceinline__ void st8(float* p, const F8& v) { st4(p, v.a); st4(p + 4, v.b); }
__device__ __forceinline__ void st8(__nv_bfloat16* p, const F8& v) {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v.a.x, v.a.y), h1 = __floats2bfloat162_rn(v.a.z, v.a.w);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(v.b.x, v.b.y), h3 = __floats2bfloat162_rn(v.b.z, v.b.w);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void add4(float4& x, const float4& y) { x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
__device__ __forceinline__ float4 shfl4(const float4& v, int m) {
    return make_float4(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m),
                       __shfl_xor_sync(0xffffffffu, v.z, m), __shfl_xor_sync(0xffffffffu, v.w, m));
}
// first half of the head: a cos - b sin; second half: a sin + b cos with a the partner
__device__ __forceinline__ float4 rotate4(const float4& x, const float4& o, const float4& c, const float4& sn, bool first) {
    if (first) return make_float4(x.x * c.x - o.x * sn.x, x.y * c.y - o.y * sn.y, x.z * c.z - o.z * sn.z, x.w * c.w - o.w * sn.w);
    return make_float4(o.x * sn.x + x.x * c.x, o.y * sn.y + x.y * c.y, o.z * sn.z + x.z * c.z, o.w * sn.w + x.w * c.w);
}

template <typename TI, typename TQ, typename TKV, int ITERS>
__global__ void qk_norm_rope_d128_wide_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                              const float* __restrict__ bias, const float* __restrict__ q_w,
                                              const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                              int max_pos, const int32_t* __restrict__ positions,
                                              const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                              TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                              int page_size, int HQ, int HKV, RowFactor rf) {
    constexpr int D = 128;
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int head0 = (blockIdx.y * WARPS + warp) * 2 * ITERS + half;      // this half-warp's heads: head0, head0 + 2, ...
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    const int d0 = l16 * 8;
    const float rs = row_factor(rf, t);
    F8 v[ITERS];
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
        v[i] = {make_float4(0.0f, 0.0f, 0.0f, 0.0f), make_float4(0.0f, 0.0f, 0.0f, 0.0f)};
        const int head = head0 + 2 * i;
        if (head >= n_heads) continue;
        const TI* src = qkv + (size_t)t * n_heads * D + (size_t)head * D + d0;
        for (int s0 = 0; s0 < splits; ++s0) {
            const F8 u = ld8(src + (size_t)s0 * split_stride);
            add4(v[i].a, u.a);
            add4(v[i].b, u.b);
        }
    }
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float4 c0 = make_float4(1.0f, 1.0f, 1.0f, 1.0f), c1 = c0, s0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), s1 = s0;
    if (cos_sin) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        const int j = (l16 & 7) * 8;                         // pair index of this lane's first dimension
        const float* row = cos_sin + (size_t)pos * D;
        c0 = ld4(row + j); c1 = ld4(row + j + 4);
        s0 = ld4(row + 64 + j); s1 = ld4(row + 64 + j + 4);
    }
    const bool first = l16 < 8;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
        const int head = head0 + 2 * i;
        const bool live = head < n_heads;                     // the shuffles below are run by every lane
        F8 x = v[i];
        x.a = make_float4(x.a.x * rs, x.a.y * rs, x.a.z * rs, x.a.w * rs);
        x.b = make_float4(x.b.x * rs, x.b.y * rs, x.b.z * rs, x.b.w * rs);
        if (bias && live) {
            const F8 b = ld8(bias + (size_t)head * D + d0);
            add4(x.a, b.a);
            add4(x.b, b.b);
        }
        const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
        const float* w = is_q ? q_w : k_w;
        // sum of squares: the two four-element groups of the lane apart over the half-warp, then together
        float p0 = x.a.x * x.a.x + x.a.y * x.a.y + x.a.z * x.a.z + x.a.w * x.a.w;
        float p1 = x.b.x * x.b.x + x.b.y * x.b.y + x.b.z * x.b.z + x.b.w * x.b.w;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            p0 += __shfl_xor_sync(0xffffffffu, p0, o);
            p1 += __shfl_xor_sync(0xffffffffu, p1, o);
        }
        F8 y = x;
        if (w && (is_q || is_k) && live) {
            const float inv = rsqrtf((p0 + p1) / (float)D + eps);
            const F8 g = ld8(w + d0);
            y.a = make_float4(x.a.x * inv * g.a.x, x.a.y * inv * g.a.y, x.a.z * inv * g.a.z, x.a.w * inv * g.a.w);
            y.b = make_float4(x.b.x * inv * g.b.x, x.b.y * inv * g.b.y, x.b.z * inv * g.b.z, x.b.w * inv * g.b.w);
        }
        const float4 oa = shfl4(y.a, 8), ob = shfl4(y.b, 8);
        if (!live) continue;
        if (!is_q && !is_k) {
            if (slot >= 0) {
                const int h = head - HQ - HKV;
                st8(v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
            }
            continue;
        }
        if (cos_sin) {
            y.a = rotate4(y.a, oa, c0, s0, first);
            y.b = rotate4(y.b, ob, c1, s1, first);
        }
        if (is_q) {
            st8(q_out + ((size_t)t * HQ + head) * D + d0, y);
        } else if (slot >= 0) {
            const int h = head - HQ;
            st8(k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, y);
        }
    }
}

}  // namespace

PH_EXPORT int ph_qk_norm_rope_kv_write(const void* qkv, int qkv_dtype, int splits, long long split_stride,
                                       const float* bias, const float* q_norm_w, const float* k_norm_w, float eps,
                                       const float* cos_sin, int n_rot, int max_pos, const int32_t* positions,
                                       const int32_t* slot_mapping, void* q_out, int q_dtype, void* k_base,
                                       void* v_base, int kv_dtype, long long page_stride, int page_size, int T,
                                       int HQ, int HKV, int D, int interleaved, const float* row_sumsq, int row_chunks,
                                       int row_width, float row_eps, cudaStream_t stream) {
    if (!qkv || !positions || !q_out || T < 0 || HQ < 1 || HKV < 0 || D < 2 || splits < 1 || !valid_dtype(qkv_dtype) ||
        !valid_dtype(q_dtype) || !valid_dtype(kv_dtype))
        return fail(PH_ERR_ARG, "qk_norm_rope: bad arguments (T %d, HQ %d, HKV %d, D %d)", T, HQ, HKV, D);
    if (D > MAX_D) return fail(PH_ERR_UNSUPPORTED, "qk_norm_rope: head_dim %d exceeds the supported %d", D, MAX_D);
    if (cos_sin && (n_rot < 2 || n_rot > D || (n_rot & 1) || max_pos < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: rotary width %d must be even and at most head_dim %d", n_rot, D);
    if (slot_mapping && (!k_base || !v_base || page_size < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: a cache write needs the pool and its page size");
    if (row_sumsq && (row_chunks < 1 || row_width < 1)) return fail(PH_ERR_ARG, "qk_norm_rope: a row factor needs its chunks and the row width");
    if (T == 0) return PH_OK;
    const RowFactor rf = {row_sumsq, row_chunks, row_width, row_eps};
    dim3 grid(T, (HQ + 2 * HKV + WARPS - 1) / WARPS);
    const bool fast = D == 128 && (!cos_sin || (n_rot == 128 && !interleaved)) && split_stride % 4 == 0 &&
                      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_base | (uintptr_t)v_base | (uintptr_t)bias |
                        (uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)cos_sin) & 15) == 0 && page_stride % 8 == 0;
    if (fast) {
        const int n_heads = HQ + 2 * HKV;
        // enough tokens to fill the device with warps that walk three pairs of heads each: the wide kernel
        const bool many = (long long)T * n_heads >= 16384 && page_stride % 8 == 0 && split_stride % 8 == 0;
        const dim3 fgrid(T, many ? (n_heads + WARPS * 6 - 1) / (WARPS * 6) : (n_heads + WARPS - 1) / WARPS);
#define LAUNCH_FAST(TI, TQ, TKV)                                                                                    \
    do {                                                                                                            \
        if (many)                                                                                                   \
            launch_overlapped(qk_norm_rope_d128_wide_kernel<TI, TQ, TKV, 3>, fgrid, dim3(WARPS * 32), 0, stream, (const TI*)qkv, \
                              splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, max_pos, positions,     \
                              slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, rf); \
        else                                                                                                        \
            launch_overlapped(qk_norm_rope_d128_kernel<TI, TQ, TKV, 1>, fgrid, dim3(WARPS * 32), 0, stream, (const TI*)qkv, \
                              splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, max_pos, positions,     \
                              slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, rf); \
    } while (0)
        PH_DISPATCH(qkv_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH_FAST(TI, TQ, TKV))));
#undef LAUNCH_FAST
        return check_launch("qk_norm_rope");
    }
#define LAUNCH(TI, TQ, TKV)                                                                                       \
    qk_norm_rope_kernel<TI, TQ, TKV><<<grid, WARPS * 32, 0, stream>>>(                                            \
        (const TI*)qkv, splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, n_rot, max_pos, positions,  \
        slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, D, interleaved, rf)
    PH_DISPATCH(qkv_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH(TI, TQ, TKV))));
#undef LAUNCH
    return check_launch("qk_norm_rope");
}

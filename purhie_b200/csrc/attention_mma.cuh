// Building blocks of the tensor-core attention kernels: cp.async and ldmatrix wrappers, the bf16
// mma.sync.m16n8k16, shared-memory tile layouts, one warp's Q K^T and P V over a tile, and the online-softmax
// update.  Used by attention_flash.cu and attention_decode_bulk.cu.
#pragma once

#include "common.cuh"

#include <math.h>

namespace ph_attn {

using namespace ph;

constexpr int BLOCK_KEYS = 64;
constexpr int THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                      // 0 bytes read: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(uint32_t*)&v;
}

// A tile of rows x D bfloat16 in shared memory, in 16-byte chunks.  Two layouts keep the 8 rows that an
// ldmatrix touches in different banks: swizzled (chunk c of row r stored at chunk c ^ (r & 7); rows D * 2
// bytes apart) for tiles filled chunk by chunk, and padded (rows D * 2 + 16 bytes apart, chunks in order) for
// tiles filled a whole row at a time by bulk copies.
template <int D, bool PAD = false> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    if constexpr (PAD) return (uint32_t)(row * (D * 2 + 16) + chunk * 16);
    else return (uint32_t)(row * (D / 8) + (chunk ^ (row & 7))) * 16u;
}

struct PagedKV {
    const __nv_bfloat16* k_base;
    const __nv_bfloat16* v_base;
    long long page_stride;
    int page_size;
    const int32_t* table;     // this request's block table
    int kv_head;
};

// Gather keys [key0, key0 + 64) of one kv head into the K and V tiles; rows outside [lo, hi] are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_block(const PagedKV& kv, int key0, int lo, int hi, uint32_t k_tile, uint32_t v_tile) {
    constexpr int CPR = D / 8;
    constexpr int ROWS_PER_PASS = THREADS / CPR;
    const int chunk = threadIdx.x % CPR;
#pragma unroll
    for (int r0 = 0; r0 < BLOCK_KEYS; r0 += ROWS_PER_PASS) {
        const int row = r0 + threadIdx.x / CPR;
        const int p = key0 + row;
        const bool valid = p >= lo && p <= hi;
        size_t off = 0;
        if (valid) {
            const int page = kv.table[p / kv.page_size];
            off = (size_t)page * kv.page_stride + ((size_t)kv.kv_head * kv.page_size + p % kv.page_size) * D + chunk * 8;
        }
        cp_async16(k_tile + tile_off<D>(row, chunk), kv.k_base + off, valid);
        cp_async16(v_tile + tile_off<D>(row, chunk), kv.v_base + off, valid);
    }
}

// One warp: S[16 x NK keys] = Q[16 x D] K^T for keys [kofs, kofs + NK) of the K tile.  qf: the warp's Q
// fragments, 4 registers per 16 dimensions.
template <int D, int NK, bool PAD = false>
__device__ __forceinline__ void warp_qk(const uint32_t (&qf)[D / 16][4], uint32_t k_tile, int kofs, float (&s)[NK / 8][4]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nt][i] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int nt = 0; nt < NK / 8; nt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = kofs + nt * 8 + (lane & 7) + ((lane >> 4) << 3);
            const int chunk = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(k_tile + tile_off<D, PAD>(row, chunk), b0, b1, b2, b3);
            mma_bf16(s[nt], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
            mma_bf16(s[nt + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
        }
    }
}

// One warp: O[16 x D] += P[16 x NK] V[NK x D] for keys [kofs, kofs + NK) of the V tile; p holds exp'd scores.
template <int D, int NK, bool PAD = false>
__device__ __forceinline__ void warp_pv(const float (&p)[NK / 8][4], uint32_t v_tile, int kofs, float (&o)[D / 8][4]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < NK / 16; ++j) {
        const uint32_t a0 = pack_bf16(p[2 * j][0], p[2 * j][1]);
        const uint32_t a1 = pack_bf16(p[2 * j][2], p[2 * j][3]);
        const uint32_t a2 = pack_bf16(p[2 * j + 1][0], p[2 * j + 1][1]);
        const uint32_t a3 = pack_bf16(p[2 * j + 1][2], p[2 * j + 1][3]);
#pragma unroll
        for (int dt = 0; dt < D / 8; dt += 2) {
            uint32_t b0, b1, b2, b3;
            const int row = kofs + j * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int chunk = dt + (lane >> 4);
            ldmatrix_x4_trans(v_tile + tile_off<D, PAD>(row, chunk), b0, b1, b2, b3);
            mma_bf16(o[dt], a0, a1, a2, a3, b0, b1);
            mma_bf16(o[dt + 1], a0, a1, a2, a3, b2, b3);
        }
    }
}

// Online softmax of one warp's scores for keys key0 + [0, NK): masks, updates (m, l) of the thread's two rows
// (lane / 4 and lane / 4 + 8), rescales o and turns s into probabilities.  z0, z1: the rows' positions.
template <int D, int NK>
__device__ __forceinline__ void softmax_update(float (&s)[NK / 8][4], int key0, int z0, int z1, int lo0, int lo1,
                                               bool need_mask, float scale_log2, float (&m)[2], float (&l)[2],
                                               float (&o)[D / 8][4]) {
    const int lane = threadIdx.x & 31;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float v = s[nt][i] * scale_log2;
            if (need_mask) {
                const int p = key0 + nt * 8 + (lane & 3) * 2 + (i & 1);
                const bool vis = (i < 2) ? (p <= z0 && p >= lo0) : (p <= z1 && p >= lo1);
                if (!vis) v = -INFINITY;
            }
            s[nt][i] = v;
            if (i < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float use0 = mn0 == -INFINITY ? 0.0f : mn0, use1 = mn1 == -INFINITY ? 0.0f : mn1;
    const float c0 = exp2f(m[0] - use0), c1 = exp2f(m[1] - use1);      // m = -inf: 0
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NK / 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - use0); s[nt][1] = exp2f(s[nt][1] - use0);
        s[nt][2] = exp2f(s[nt][2] - use1); s[nt][3] = exp2f(s[nt][3] - use1);
        sum0 += s[nt][0] + s[nt][1];
        sum1 += s[nt][2] + s[nt][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l[0] = l[0] * c0 + sum0;
    l[1] = l[1] * c1 + sum1;
    m[0] = mn0;
    m[1] = mn1;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= c0; o[dt][1] *= c0;
        o[dt][2] *= c1; o[dt][3] *= c1;
    }
}

}  // namespace ph_attn

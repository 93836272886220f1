// Attention over cache pages on the tensor cores (bfloat16 in, float32 softmax and accumulation):
//   * attention_prefill: portions of prompts.  One CTA per (64 query tokens of one request, query head);
//     keys are walked in blocks of 64 from the first visible one to the diagonal (flash attention: running
//     maximum and sum per row, the output rescaled as the maximum moves).
//   * attention_decode: single tokens.  One CTA per (token, kv head, split of the keys): the HQ / HKV query
//     heads that share the kv head form the rows of one 16-row tile, the four warps of the CTA take 16 keys
//     each of every 64-key block, and the CTA leaves (maximum, sum, unnormalised output) per head;
//   * attention_combine merges the splits in a fixed order.
// Keys and values are gathered from pages with 16-byte cp.async copies into swizzled shared memory, two
// blocks in flight; rows outside the visible range are zero-filled, so whatever an unwritten or reused page
// holds (NaN included) never reaches a product.  A row at absolute position z sees positions
// max(0, z - window + 1) .. z (window 0: all of them).
// Math as in the reference: src/attention.hip:612-701 (flash tiles, online softmax), :315-443 (partial
// results per chunk and their combination), scale 1/sqrt(D) applied to the scores (src/attention.cpp:197).
#include "attention_mma.cuh"

namespace {

using namespace ph;
using namespace ph_attn;

// ---- prefill ---------------------------------------------------------------------------------------------

template <int D>
__global__ void __launch_bounds__(THREADS) attention_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_base, const __nv_bfloat16* __restrict__ v_base,
    long long page_stride, int page_size, const int32_t* __restrict__ block_table, int table_stride,
    const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_ctx_len, const int32_t* __restrict__ tile_seg,
    const int32_t* __restrict__ tile_first, __nv_bfloat16* __restrict__ out, int HQ, int HKV, int window, float scale_log2) {
    constexpr int BM = 64;
    constexpr int TILE_BYTES = BLOCK_KEYS * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);
    const uint32_t kv_tiles = q_tile + BM * D * 2;            // [2 buffers][K, V]

    const int tile = blockIdx.y, h = blockIdx.x;                   // heads of one tile start together; the caller lists long tiles first
    const int seg = tile_seg[tile], first = tile_first[tile];      // first: index of the tile's first token in its portion
    const int row0 = seg_start[seg], q_len = seg_start[seg + 1] - row0;
    const int ctx_len = seg_ctx_len[seg];
    const int n_rows = min(BM, q_len - first);
    const int z_first = ctx_len - q_len + first;                    // absolute position of the tile's first row
    const int z_last = z_first + n_rows - 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    PagedKV kv{k_base, v_base, page_stride, page_size, block_table + (size_t)seg * table_stride, h / (HQ / HKV)};

    // Q tile: rows beyond the portion are zero
    {
        constexpr int CPR = D / 8;
        const int chunk = threadIdx.x % CPR;
        for (int r = threadIdx.x / CPR; r < BM; r += THREADS / CPR) {
            const bool valid = r < n_rows;
            const __nv_bfloat16* src = q + ((size_t)(row0 + first + (valid ? r : 0)) * HQ + h) * D + chunk * 8;
            cp_async16(q_tile + tile_off<D>(r, chunk), src, valid);
        }
    }
    const int lo_tile = window > 0 ? max(0, z_first - window + 1) : 0;
    const int kb_first = lo_tile / BLOCK_KEYS, kb_last = z_last / BLOCK_KEYS;
    load_kv_block<D>(kv, kb_first * BLOCK_KEYS, lo_tile, z_last, kv_tiles, kv_tiles + TILE_BYTES);
    cp_async_commit();

    // this thread's two rows
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int z0 = z_first + min(r0, n_rows - 1), z1 = z_first + min(r1, n_rows - 1);
    const int lo0 = window > 0 ? max(0, z0 - window + 1) : 0, lo1 = window > 0 ? max(0, z1 - window + 1) : 0;
    const int warp_zmin = z_first + min(warp * 16, n_rows - 1), warp_zmax = z_first + min(warp * 16 + 15, n_rows - 1);
    const int warp_lomax = window > 0 ? max(0, warp_zmax - window + 1) : 0;

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int buf = (kb - kb_first) & 1;
        const uint32_t k_tile = kv_tiles + buf * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
        if (kb < kb_last) {
            const uint32_t nk = kv_tiles + (buf ^ 1) * 2 * TILE_BYTES;
            load_kv_block<D>(kv, (kb + 1) * BLOCK_KEYS, lo_tile, z_last, nk, nk + TILE_BYTES);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kb == kb_first) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(q_tile + tile_off<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        const int key0 = kb * BLOCK_KEYS;
        // a warp skips blocks none of its rows can see
        if (key0 <= warp_zmax && key0 + BLOCK_KEYS - 1 >= (window > 0 ? max(0, warp_zmin - window + 1) : 0)) {
            float s[BLOCK_KEYS / 8][4];
            warp_qk<D, BLOCK_KEYS>(qf, k_tile, 0, s);
            const bool need_mask = key0 + BLOCK_KEYS - 1 > warp_zmin || key0 < warp_lomax;
            softmax_update<D, BLOCK_KEYS>(s, key0, z0, z1, lo0, lo1, need_mask, scale_log2, m, l, o);
            warp_pv<D, BLOCK_KEYS>(s, v_tile, 0, o);
        }
        __syncthreads();
    }
    const float inv0 = l[0] == 0.0f ? 0.0f : 1.0f / l[0], inv1 = l[1] == 0.0f ? 0.0f : 1.0f / l[1];
    const size_t width = (size_t)HQ * D;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
        if (r0 < n_rows)
            *(uint32_t*)(out + (size_t)(row0 + first + r0) * width + (size_t)h * D + d) = pack_bf16(o[dt][0] * inv0, o[dt][1] * inv0);
        if (r1 < n_rows)
            *(uint32_t*)(out + (size_t)(row0 + first + r1) * width + (size_t)h * D + d) = pack_bf16(o[dt][2] * inv1, o[dt][3] * inv1);
    }
}

// ---- decode ----------------------------------------------------------------------------------------------

// Partial results: part_o [rows][HQ][splits][D] float32 (unnormalised), part_ml [rows][HQ][splits][2] = (m, l),
// m in the log2 domain (scores * scale * log2 e).
template <int D>
__global__ void __launch_bounds__(THREADS) attention_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_base, const __nv_bfloat16* __restrict__ v_base,
    long long page_stride, int page_size, const int32_t* __restrict__ block_table, int table_stride,
    const int32_t* __restrict__ row_list, const int32_t* __restrict__ row_seg, const int32_t* __restrict__ positions,
    float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int HQ, int HKV, int splits,
    int window, float scale_log2) {
    constexpr int TILE_BYTES = BLOCK_KEYS * D * 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t q_tile = smem_u32(smem);                     // 16 x D
    const uint32_t kv_tiles = q_tile + 16 * D * 2;
    float* red = (float*)(smem + 16 * D * 2);                    // after the loop: [4 warps][16 rows][D + 2]

    const int t = row_list ? row_list[blockIdx.x] : blockIdx.x;
    const int g = blockIdx.y, split = blockIdx.z;
    const int G = HQ / HKV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int z = positions[t];
    const int lo = window > 0 ? max(0, z - window + 1) : 0;
    const int n_blocks = (z - lo) / BLOCK_KEYS + 1;
    const int per = (n_blocks + splits - 1) / splits;
    const int b_first = split * per, b_last = min(n_blocks, b_first + per) - 1;

    PagedKV kv{k_base, v_base, page_stride, page_size, block_table + (size_t)row_seg[t] * table_stride, g};

    {   // Q: the G heads of this kv head are rows 0 .. G-1, the rest is zero
        constexpr int CPR = D / 8;
        for (int idx = threadIdx.x; idx < 16 * CPR; idx += THREADS) {
            const int r = idx / CPR, chunk = idx % CPR;
            const bool valid = r < G;
            const __nv_bfloat16* src = q + ((size_t)t * HQ + (size_t)g * G + (valid ? r : 0)) * D + chunk * 8;
            cp_async16(q_tile + tile_off<D>(r, chunk), src, valid);
        }
    }
    if (b_first <= b_last) load_kv_block<D>(kv, lo + b_first * BLOCK_KEYS, lo, z, kv_tiles, kv_tiles + TILE_BYTES);
    cp_async_commit();

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;

    for (int b = b_first; b <= b_last; ++b) {
        const int buf = (b - b_first) & 1;
        const uint32_t k_tile = kv_tiles + buf * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
        if (b < b_last) {
            const uint32_t nk = kv_tiles + (buf ^ 1) * 2 * TILE_BYTES;
            load_kv_block<D>(kv, lo + (b + 1) * BLOCK_KEYS, lo, z, nk, nk + TILE_BYTES);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (b == b_first) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(q_tile + tile_off<D>(lane & 15, ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        const int key0 = lo + b * BLOCK_KEYS + warp * 16;           // this warp's 16 keys of the block
        if (key0 <= z) {
            float s[2][4];
            warp_qk<D, 16>(qf, k_tile, warp * 16, s);
            softmax_update<D, 16>(s, key0, z, z, lo, lo, key0 + 15 > z, scale_log2, m, l, o);
            warp_pv<D, 16>(s, v_tile, warp * 16, o);
        }
        __syncthreads();
    }
    // merge the four warps (each saw different keys); rows >= G are padding
    cp_async_wait<0>();
    __syncthreads();
    constexpr int RS = D + 2;
    const int r0 = lane >> 2, r1 = r0 + 8;
    float* mine = red + (size_t)warp * 16 * RS;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
        mine[r0 * RS + d] = o[dt][0]; mine[r0 * RS + d + 1] = o[dt][1];
        mine[r1 * RS + d] = o[dt][2]; mine[r1 * RS + d + 1] = o[dt][3];
    }
    if ((lane & 3) == 0) {
        mine[r0 * RS + D] = m[0]; mine[r0 * RS + D + 1] = l[0];
        mine[r1 * RS + D] = m[1]; mine[r1 * RS + D + 1] = l[1];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += THREADS) {
        const int r = idx / D, d = idx % D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[((size_t)w * 16 + r) * RS + D]);
        const float use = mm == -INFINITY ? 0.0f : mm;
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = red + ((size_t)w * 16 + r) * RS;
            const float c = exp2f(src[D] - use);
            acc += c * src[d];
            ll += c * src[D + 1];
        }
        const int h = g * G + r;
        if (splits == 1) {
            out[((size_t)t * HQ + h) * D + d] = __float2bfloat16_rn(ll == 0.0f ? 0.0f : acc / ll);
        } else {
            const size_t slot = ((size_t)blockIdx.x * HQ + h) * splits + split;
            part_o[slot * D + d] = acc;
            if (d == 0) { part_ml[slot * 2] = mm; part_ml[slot * 2 + 1] = ll; }
        }
    }
}

template <int D>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         const int32_t* __restrict__ row_list, __nv_bfloat16* __restrict__ out, int HQ, int splits) {
    const int i = blockIdx.x, h = blockIdx.y;
    const int t = row_list ? row_list[i] : i;
    const size_t slot0 = ((size_t)i * HQ + h) * splits;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(slot0 + s) * 2]);
    const float use = mm == -INFINITY ? 0.0f : mm;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f, ll = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float c = exp2f(part_ml[(slot0 + s) * 2] - use);
            acc += c * part_o[(slot0 + s) * D + d];
            ll += c * part_ml[(slot0 + s) * 2 + 1];
        }
        out[((size_t)t * HQ + h) * D + d] = __float2bfloat16_rn(ll == 0.0f ? 0.0f : acc / ll);
    }
}

// Raise a kernel's dynamic shared-memory limit, once per kernel and device (TAG tells kernels of one signature
// apart; the attribute belongs to the kernel as loaded on one device).
template <int TAG, typename K> int set_smem(K kernel, int bytes) {
    static bool done[64] = {false};
    if (bytes <= 48 * 1024) return PH_OK;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (done[dev]) return PH_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
        return fail(PH_ERR_LAUNCH, "attention_flash: cannot reserve %d bytes of shared memory", bytes);
    done[dev] = true;
    return PH_OK;
}

}  // namespace

PH_DEFINE_LAST_ERROR(ph_flash)

PH_EXPORT int ph_attention_prefill(const void* q, const void* k_base, const void* v_base, long long page_stride,
                                   int page_size, const int32_t* block_table, int table_stride, const int32_t* seg_start,
                                   const int32_t* seg_ctx_len, const int32_t* tile_seg, const int32_t* tile_first,
                                   int n_tiles, void* out, int HQ, int HKV, int D, int window, float scale,
                                   cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !seg_start || !seg_ctx_len || !tile_seg || !tile_first || !out ||
        n_tiles < 0 || HQ < 1 || HKV < 1 || HQ % HKV || page_size < 1 || window < 0)
        return fail(PH_ERR_ARG, "attention_prefill: bad arguments (tiles %d, HQ %d, HKV %d)", n_tiles, HQ, HKV);
    if (D != 64 && D != 128) return fail(PH_ERR_UNSUPPORTED, "attention_prefill: head_dim %d is not 64 or 128", D);
    if (n_tiles > 65535) return fail(PH_ERR_UNSUPPORTED, "attention_prefill: %d tiles exceed the grid", n_tiles);
    if (n_tiles == 0) return PH_OK;
    const float scale_log2 = scale * LOG2E;
    dim3 grid(HQ, n_tiles);
#define LAUNCH(DD)                                                                                               \
    do {                                                                                                         \
        const int bytes = 64 * DD * 2 + 4 * BLOCK_KEYS * DD * 2;                                                 \
        if (int rc = set_smem<2 * DD>(attention_prefill_kernel<DD>, bytes)) return rc;                                   \
        attention_prefill_kernel<DD><<<grid, THREADS, bytes, stream>>>(                                          \
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_base, (const __nv_bfloat16*)v_base, page_stride,    \
            page_size, block_table, table_stride, seg_start, seg_ctx_len, tile_seg, tile_first,                  \
            (__nv_bfloat16*)out, HQ, HKV, window, scale_log2);                                                   \
    } while (0)
    if (D == 64) LAUNCH(64); else LAUNCH(128);
#undef LAUNCH
    return check_launch("attention_prefill");
}

PH_EXPORT int ph_attention_decode(const void* q, const void* k_base, const void* v_base, long long page_stride,
                                  int page_size, const int32_t* block_table, int table_stride, const int32_t* row_list,
                                  int n_rows, const int32_t* row_seg, const int32_t* positions, float* part_o,
                                  float* part_ml, void* out, int HQ, int HKV, int D, int splits, int window, float scale,
                                  cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !row_seg || !positions || !out || n_rows < 0 || HQ < 1 || HKV < 1 ||
        HQ % HKV || page_size < 1 || window < 0 || splits < 1 || (splits > 1 && (!part_o || !part_ml)))
        return fail(PH_ERR_ARG, "attention_decode: bad arguments (rows %d, HQ %d, HKV %d, splits %d)", n_rows, HQ, HKV, splits);
    if (D != 64 && D != 128) return fail(PH_ERR_UNSUPPORTED, "attention_decode: head_dim %d is not 64 or 128", D);
    if (HQ / HKV > 16) return fail(PH_ERR_UNSUPPORTED, "attention_decode: %d query heads per kv head exceed 16", HQ / HKV);
    if (HKV > 65535 || splits > 65535) return fail(PH_ERR_UNSUPPORTED, "attention_decode: grid too large");
    if (n_rows == 0) return PH_OK;
    const float scale_log2 = scale * LOG2E;
    dim3 grid(n_rows, HKV, splits);
#define LAUNCH(DD)                                                                                               \
    do {                                                                                                         \
        const int kv_bytes = 4 * BLOCK_KEYS * DD * 2, red_bytes = 4 * 16 * (DD + 2) * 4;                         \
        const int bytes = 16 * DD * 2 + (kv_bytes > red_bytes ? kv_bytes : red_bytes);                           \
        if (int rc = set_smem<2 * DD + 1>(attention_decode_kernel<DD>, bytes)) return rc;                                    \
        attention_decode_kernel<DD><<<grid, THREADS, bytes, stream>>>(                                           \
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_base, (const __nv_bfloat16*)v_base, page_stride,    \
            page_size, block_table, table_stride, row_list, row_seg, positions, part_o, part_ml,                 \
            (__nv_bfloat16*)out, HQ, HKV, splits, window, scale_log2);                                           \
        if (splits > 1)                                                                                          \
            attention_combine_kernel<DD><<<dim3(n_rows, HQ), DD < 128 ? DD : 128, 0, stream>>>(                  \
                part_o, part_ml, row_list, (__nv_bfloat16*)out, HQ, splits);                                     \
    } while (0)
    if (D == 64) LAUNCH(64); else LAUNCH(128);
#undef LAUNCH
    return check_launch("attention_decode");
}

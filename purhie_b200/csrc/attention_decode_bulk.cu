// Decode attention as a persistent, warp-specialised kernel fed by TMA.
//
// One CTA per SM walks over work items (token, kv head, split of the keys).  A producer warp copies whole pages
// into a ring of stages of 64 keys: ONE TMA box per page brings the page's keys and values of the kv head
// (4-D box: 64 elements x page_size rows x head_dim / 64 halves x {K, V}, 128-byte swizzled by the copy engine),
// completion counted on an mbarrier per stage, and the producer runs ahead of the consumers across items, so
// the memory system stays busy while a finished item is merged and written.  Four consumer
// warps take 16 keys each of every stage: Q K^T and P V on mma.sync.m16n8k16 with the group's query heads as the
// 16-row tile, online softmax in float32; per item the four warps' results are merged through shared memory and
// stored as a partial result (maximum, sum, unnormalised output) per split, or as the final output when there
// is one split.
// What a token may not see never reaches a product: pages beyond its position are fetched from an
// out-of-range coordinate (the copy engine fills zeros), scores of invisible keys are replaced by -inf, and the
// value rows after the token's position inside its last page are zeroed in shared memory before P V, so
// unwritten page slots may hold anything, NaN included.  Every mbarrier wait is bounded and reports through an
// error word.  The math is that of attention_flash.cu's decode kernel.
#include "attention_mma.cuh"
#include "mbarrier.cuh"

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace ph;
using namespace ph_attn;
namespace mb = ph_mbar;

constexpr int CONSUMER_WARPS = 4;
constexpr int BULK_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int PAGE_CACHE = 256;

#define PH_ERR_WAIT_ATTN_PRODUCER 111
#define PH_ERR_WAIT_ATTN_CONSUMER 112

struct BulkParams {
    const __nv_bfloat16* q;
    long long rows_per_page;       // page_stride / D: rows of the [rows, D] view between two pages
    int total_rows;                // rows of that view; a coordinate >= total_rows reads zeros
    int page_size, page_shift;     // page_size = 1 << page_shift
    const int32_t* block_table;
    int table_stride;
    const int32_t* row_list;
    const int32_t* row_seg;
    const int32_t* positions;
    float* part_o;
    float* part_ml;
    __nv_bfloat16* out;
    int n_rows, HQ, HKV, splits, window;
    float scale_log2;
    int* error_flag;
};

struct Item {
    int i, t, g, split, z, lo, lo_page, b_first, b_last, n_blocks;
};

// Blocks of 64 keys start at the page that holds the first visible key, so a block is a whole number of pages.
__device__ __forceinline__ Item make_item(const BulkParams& p, int w) {
    Item it;
    it.split = w % p.splits;
    const int rest = w / p.splits;
    it.g = rest % p.HKV;
    it.i = rest / p.HKV;
    it.t = p.row_list ? p.row_list[it.i] : it.i;
    it.z = p.positions[it.t];
    it.lo = p.window > 0 ? max(0, it.z - p.window + 1) : 0;
    it.lo_page = it.lo - it.lo % p.page_size;
    const int n_blocks = (it.z - it.lo_page) / BLOCK_KEYS + 1;
    it.n_blocks = n_blocks;
    const int per = (n_blocks + p.splits - 1) / p.splits;
    it.b_first = it.split * per;
    it.b_last = min(n_blocks, it.b_first + per) - 1;
    return it;
}

// One box: all of a page that belongs to one kv head, keys and values.
__device__ __forceinline__ void tma_load_page(void* dst, const CUtensorMap* map, uint64_t* bar, int row) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %3, %3}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(0), "r"(row) : "memory");
}

// A stage holds 64 keys as 64 / page_size page blocks; a page block is laid out as the box arrives:
// [K, V][half of 64 elements][row in page][128 bytes], every 128-byte row swizzled (chunk ^ (row & 7)).
// Byte offset of the 16-byte chunk `chunk` of key `row` (0 .. 63), keys (is_v 0) or values (1).
template <int D> __device__ __forceinline__ uint32_t stage_off(int row, int chunk, int is_v, int page_size, int page_shift) {
    constexpr int HALVES = D / 64;
    const int region = page_size * 128;                   // one half of one page
    return (uint32_t)((row >> page_shift) * (2 * HALVES * region) + (is_v * HALVES + (chunk >> 3)) * region +
                      (row & (page_size - 1)) * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Shared memory a CTA needs for G query heads per kv head and a ring of `stages` stages.
__host__ __device__ constexpr int bulk_smem_bytes(int D, int G, int stages) {
    return 1024 /* alignment */ + stages * 2 * BLOCK_KEYS * D * 2 + 2 * G * D * 2 + CONSUMER_WARPS * G * (D + 2) * 4 +
           (2 * stages + 4) * 8 + PAGE_CACHE * 4;
}

template <int D, int STAGES, int CTAS>
__global__ void __launch_bounds__(BULK_THREADS, CTAS)
attention_decode_bulk_kernel(const __grid_constant__ CUtensorMap map_kv, const BulkParams p) {
    constexpr int HALVES = D / 64;
    constexpr int TILE = BLOCK_KEYS * D * 2;              // bytes of K (or of V) for 64 keys
    constexpr int QROW = D * 2;
    constexpr int RS = D + 2;
    const int G = p.HQ / p.HKV;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* kv = smem;                             // [STAGES][page blocks of K and V], 1024-byte aligned
    unsigned char* q_tiles = kv + STAGES * 2 * TILE;      // [2][G rows x D]
    float* red = (float*)(q_tiles + 2 * G * QROW);        // [4 warps][G][D + 2]
    uint64_t* full = (uint64_t*)(red + CONSUMER_WARPS * G * RS);
    uint64_t* empty = full + STAGES;
    uint64_t* q_full = empty + STAGES;
    uint64_t* q_empty = q_full + 2;
    int32_t* pages = (int32_t*)(q_empty + 2);             // [PAGE_CACHE] the producer's copy of the item's block table

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int work_total = p.n_rows * p.HKV * p.splits;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mb::init(&full[s], 1); mb::init(&empty[s], CONSUMER_WARPS); }
        for (int s = 0; s < 2; ++s) { mb::init(&q_full[s], 1); mb::init(&q_empty[s], CONSUMER_WARPS); }
        mb::fence_init();
    }
    pdl_launch_dependents();
    __syncthreads();
    // The queries and this step's keys and values come from the kernel before this one: the consumers wait for
    // it here, the producer only after it has requested what older steps wrote (below).
    if (warp != CONSUMER_WARPS) pdl_wait();

    if (warp == CONSUMER_WARPS) {
        // ---- producer ----
        // All lanes run the same control flow: lane 0 waits on the barriers and announces the bytes, lane j
        // issues the box of the stage's page j.  The box coordinates of the whole item are worked out by all lanes
        // at once when the item starts, so that a stage costs the producer a few instructions.
        int stage = 0, qi = 0;
        uint32_t phase = 0, q_phase = 0;
        int ok = 1;
        const int psh = p.page_shift, ppb = BLOCK_KEYS >> psh;              // pages per stage
        const int page_block = 2 * HALVES * p.page_size * 128;             // bytes of one page's box
        bool waited = false;                                                // for the kernel in front
        for (int w = blockIdx.x; w < work_total && ok; w += gridDim.x) {
            const Item it = make_item(p, w);
            const int32_t* table = p.block_table + (size_t)p.row_seg[it.t] * p.table_stride;
            const int nb = it.b_last - it.b_first + 1;
            const int key_first = it.lo_page + it.b_first * BLOCK_KEYS;
            // row coordinate of page j of the item: its place in the pool, or out of range (zeros) past the token
            auto page_row = [&](int j) {
                const int pos = key_first + (j << psh);
                if (pos > it.z) return p.total_rows;
                return (int)((long long)table[pos >> psh] * p.rows_per_page + (long long)it.g * p.page_size);
            };
            __syncwarp();                                                    // the previous item's boxes are issued
            for (int j = lane; j < nb * ppb && j < PAGE_CACHE; j += 32) pages[j] = page_row(j);
            __syncwarp();
            // The first item's leading blocks hold keys and values of earlier steps (block tables and positions were
            // uploaded before the step began): they are requested while the kernel in front still runs.  The block
            // with the token's own position, the row's last (whichever split it falls to), is not among them.
            int b_start = 0;
            if (!waited) {
                int n_pre = min(nb, STAGES);
                if (it.b_last == it.n_blocks - 1) n_pre = min(n_pre, nb - 1);
                for (; b_start < n_pre; ++b_start) {
                    if (lane == 0) mb::arrive_expect_tx(&full[stage], 2 * TILE);      // the ring is still empty
                    __syncwarp();
                    if (lane < ppb) {
                        const int j = b_start * ppb + lane;
                        tma_load_page(kv + stage * 2 * TILE + lane * page_block, &map_kv, &full[stage], j < PAGE_CACHE ? pages[j] : page_row(j));
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                pdl_wait();
                waited = true;
            }
            // the query rows of this kv head's group are contiguous: one copy
            if (lane == 0) {
                ok = mb::wait(&q_empty[qi], q_phase ^ 1, p.error_flag, PH_ERR_WAIT_ATTN_PRODUCER) ? 1 : 0;
                if (ok) {
                    mb::arrive_expect_tx(&q_full[qi], G * QROW);
                    mb::bulk_copy(q_tiles + qi * G * QROW, p.q + ((size_t)it.t * p.HQ + (size_t)it.g * G) * D, G * QROW, &q_full[qi]);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (++qi == 2) { qi = 0; q_phase ^= 1; }
            for (int b = b_start; b < nb; ++b) {
                if (lane == 0) {
                    ok = mb::wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_ATTN_PRODUCER) ? 1 : 0;
                    if (ok) mb::arrive_expect_tx(&full[stage], 2 * TILE);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);                        // also: the stage is free for every lane
                if (!ok) break;
                if (lane < ppb) {
                    const int j = b * ppb + lane;
                    const int row = j < PAGE_CACHE ? pages[j] : page_row(j);
                    tma_load_page(kv + stage * 2 * TILE + lane * page_block, &map_kv, &full[stage], row);
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!waited) pdl_wait();                                            // a CTA without work
        if (lane == 0 && ok) {
            // do not leave while copies may be in flight: wait until the consumers released every stage
            for (int s = 0; s < STAGES; ++s) {
                if (!mb::wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_ATTN_PRODUCER)) break;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            for (int s = 0; s < 2; ++s) {
                if (!mb::wait(&q_empty[qi], q_phase ^ 1, p.error_flag, PH_ERR_WAIT_ATTN_PRODUCER)) break;
                if (++qi == 2) { qi = 0; q_phase ^= 1; }
            }
        }
    } else {
        // ---- consumers ----
        int stage = 0, qi = 0;
        uint32_t phase = 0, q_phase = 0;
        bool ok = true;
        const int r0 = lane >> 2, r1 = r0 + 8;
        const int ps = p.page_size, psh = p.page_shift;
        float* mine = red + (size_t)warp * G * RS;

        // S = Q K^T over this warp's 16 keys of a stage; even and odd steps of D accumulate apart, so that four
        // chains of dependent instructions run instead of two.
        auto qk = [&](uint32_t st, const uint32_t (&qf)[D / 16][4], float (&s)[2][4]) {
            float s2[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) { s[nt][i] = 0.0f; s2[nt][i] = 0.0f; }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t b0, b1, b2, b3;
                const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int chunk = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(st + stage_off<D>(row, chunk, 0, ps, psh), b0, b1, b2, b3);
                if (ks & 1) {
                    mma_bf16(s2[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma_bf16(s2[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
                } else {
                    mma_bf16(s[0], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma_bf16(s[1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[nt][i] += s2[nt][i];
        };
        // O += P V over the same 16 keys
        auto pv = [&](uint32_t st, const float (&s)[2][4], float (&o)[D / 8][4]) {
            const uint32_t a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
            const uint32_t a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int dt = 0; dt < D / 8; dt += 2) {
                uint32_t b0, b1, b2, b3;
                const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                ldmatrix_x4_trans(st + stage_off<D>(row, dt + (lane >> 4), 1, ps, psh), b0, b1, b2, b3);
                mma_bf16(o[dt], a0, a1, a2, a3, b0, b1);
                mma_bf16(o[dt + 1], a0, a1, a2, a3, b2, b3);
            }
        };

        for (int w = blockIdx.x; w < work_total && ok; w += gridDim.x) {
            const Item it = make_item(p, w);
            uint32_t qf[D / 16][4];
            if (!mb::wait(&q_full[qi], q_phase, p.error_flag, PH_ERR_WAIT_ATTN_CONSUMER)) { ok = false; break; }
            {   // the tile's rows beyond the group repeat a real row; their results are never stored
                const uint32_t q_tile = smem_u32(q_tiles + qi * G * QROW);
                const int qrow = min(lane & 15, G - 1);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    ldmatrix_x4(q_tile + qrow * QROW + (ks * 2 + (lane >> 4)) * 16, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            }
            const int q_used = qi;                          // given back after the item's last block, see below
            if (++qi == 2) { qi = 0; q_phase ^= 1; }

            float o[D / 8][4];
            float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
                for (int i = 0; i < 4; ++i) o[dt][i] = 0.0f;

            // The scores of block j + 1 are computed in the same straight-line code as the softmax and P V of
            // block j, so that the scheduler can overlap the two dependency chains.
            const int nb = it.b_last - it.b_first + 1;
            float s_cur[2][4];
            if (nb > 0) {
                if (!mb::wait(&full[stage], phase, p.error_flag, PH_ERR_WAIT_ATTN_CONSUMER)) { ok = false; break; }
                qk(smem_u32(kv + stage * 2 * TILE), qf, s_cur);
            }
            for (int j = 0; j < nb; ++j) {
                unsigned char* st_ptr = kv + stage * 2 * TILE;
                const uint32_t st = smem_u32(st_ptr);
                const int key0 = it.lo_page + (it.b_first + j) * BLOCK_KEYS + warp * 16;
                int nstage = stage + 1;
                uint32_t nphase = phase;
                if (nstage == STAGES) { nstage = 0; nphase ^= 1; }
                if (j + 1 < nb) {
                    if (!mb::wait(&full[nstage], nphase, p.error_flag, PH_ERR_WAIT_ATTN_CONSUMER)) { ok = false; break; }
                    float s_next[2][4];
                    qk(smem_u32(kv + nstage * 2 * TILE), qf, s_next);
                    // not the item's last block: every key is at or before the token; only the window's start masks
                    softmax_update<D, 16>(s_cur, key0, it.z, it.z, it.lo, it.lo, true, p.scale_log2, m, l, o);
                    pv(st, s_cur, o);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) s_cur[nt][i] = s_next[nt][i];
                } else if (key0 <= it.z) {
                    const bool tail = key0 + 15 > it.z;
                    if (tail) {
                        // value rows after the token's position inside its page may hold anything: zero this warp's
                        for (int idx = lane; idx < 16 * (D / 8); idx += 32) {
                            const int r = idx / (D / 8), c = idx % (D / 8);
                            if (key0 + r > it.z) *(uint4*)(st_ptr + stage_off<D>(warp * 16 + r, c, 1, ps, psh)) = make_uint4(0, 0, 0, 0);
                        }
                        __syncwarp();
                    }
                    softmax_update<D, 16>(s_cur, key0, it.z, it.z, it.lo, it.lo, true, p.scale_log2, m, l, o);
                    pv(st, s_cur, o);
                    if (tail) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // our zeros, before the next copy lands there
                }
                __syncwarp();
                if (lane == 0) mb::arrive(&empty[stage]);
                stage = nstage;
                phase = nphase;
            }
            if (!ok) break;
            // The query buffer is given back only now: the compiler is free to fetch the fragments again from
            // shared memory inside the loop instead of keeping them in registers, so the buffer must not change
            // while the item runs.
            __syncwarp();
            if (lane == 0) mb::arrive(&q_empty[q_used]);
            // merge the four warps (each saw different keys); fragment rows >= G are padding
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt) {
                const int d = dt * 8 + (lane & 3) * 2;
                if (r0 < G) { mine[r0 * RS + d] = o[dt][0]; mine[r0 * RS + d + 1] = o[dt][1]; }
                if (r1 < G) { mine[r1 * RS + d] = o[dt][2]; mine[r1 * RS + d + 1] = o[dt][3]; }
            }
            if ((lane & 3) == 0) {
                if (r0 < G) { mine[r0 * RS + D] = m[0]; mine[r0 * RS + D + 1] = l[0]; }
                if (r1 < G) { mine[r1 * RS + D] = m[1]; mine[r1 * RS + D + 1] = l[1]; }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            for (int idx = threadIdx.x; idx < G * D; idx += CONSUMER_WARPS * 32) {
                const int r = idx / D, d = idx % D;
                float mm = -INFINITY;
#pragma unroll
                for (int ww = 0; ww < CONSUMER_WARPS; ++ww) mm = fmaxf(mm, red[((size_t)ww * G + r) * RS + D]);
                const float use = mm == -INFINITY ? 0.0f : mm;
                float acc = 0.0f, ll = 0.0f;
#pragma unroll
                for (int ww = 0; ww < CONSUMER_WARPS; ++ww) {
                    const float* src = red + ((size_t)ww * G + r) * RS;
                    const float c = exp2f(src[D] - use);
                    acc += c * src[d];
                    ll += c * src[D + 1];
                }
                const int h = it.g * G + r;
                if (p.splits == 1) {
                    p.out[((size_t)it.t * p.HQ + h) * D + d] = __float2bfloat16_rn(ll == 0.0f ? 0.0f : acc / ll);
                } else {
                    const size_t slot = ((size_t)it.i * p.HQ + h) * p.splits + it.split;
                    p.part_o[slot * D + d] = acc;
                    if (d == 0) { p.part_ml[slot * 2] = mm; p.part_ml[slot * 2 + 1] = ll; }
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");     // red is free again
        }
    }
}

template <int D>
__global__ void attention_combine_bulk_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int32_t* __restrict__ row_list, __nv_bfloat16* __restrict__ out, int HQ, int splits) {
    // One block per (row, head), a thread per element of the head.  Lane s of every warp fetches the maximum and sum
    // of split s, so that the weights of 32 splits cost one round trip, and the partial outputs are fetched eight
    // splits at a time; the sums run over the splits in ascending order whatever the block's shape.
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31;
    const int t = row_list ? row_list[i] : i;
    const size_t slot0 = ((size_t)i * HQ + h) * splits;
    float mm = -INFINITY;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        float m = s0 + lane < splits ? part_ml[(slot0 + s0 + lane) * 2] : -INFINITY;
#pragma unroll
        for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
        mm = fmaxf(mm, m);
    }
    const float use = mm == -INFINITY ? 0.0f : mm;
    const int d = threadIdx.x;                              // blockDim.x == min(D, 128); D <= 128 here
    float acc = 0.0f, ll = 0.0f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        const int n = min(32, splits - s0);
        float c = 0.0f, cl = 0.0f;
        if (lane < n) {
            c = exp2f(part_ml[(slot0 + s0 + lane) * 2] - use);
            cl = c * part_ml[(slot0 + s0 + lane) * 2 + 1];
        }
        const float* po = part_o + (slot0 + s0) * D + d;
        for (int j = 0; j < n; j += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = j + u < n ? po[(size_t)(j + u) * D] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc += __shfl_sync(0xffffffffu, c, (j + u) & 31) * v[u];      // lanes >= n hold zero
                ll += __shfl_sync(0xffffffffu, cl, (j + u) & 31);
            }
        }
    }
    out[((size_t)t * HQ + h) * D + d] = __float2bfloat16_rn(ll == 0.0f ? 0.0f : acc / ll);
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// The keys and values of one cache entry as a 4-D tensor from the entry's first key element: 64 elements, rows
// (D * 2 bytes apart), halves of a row (128 bytes apart), {K, V} (kv_stride bytes apart).  A box is one page of
// one kv head, keys and values: {64, page_size, D / 64, 2}, 128-byte swizzled, zeros outside.
bool make_page_map(CUtensorMap* out, const void* k_base, long long kv_stride_bytes, long long rows, int D, int page_size) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, long long, long long, int, int>, CUtensorMap> cache;
    const auto key = std::make_tuple(k_base, kv_stride_bytes, rows, D, page_size);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {64, (cuuint64_t)rows, (cuuint64_t)(D / 64), 2};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, 128, (cuuint64_t)kv_stride_bytes};
    const cuuint32_t box[4] = {64, (cuuint32_t)page_size, (cuuint32_t)(D / 64), 2};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(k_base), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
}

template <int D, int STAGES, int CTAS>
int launch_config(const CUtensorMap& mkv, const BulkParams& p, int bytes, int max_ctas, cudaStream_t stream) {
    static int configured = 0;
    auto kernel = attention_decode_bulk_kernel<D, STAGES, CTAS>;
    if (configured < bytes) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
            return fail(PH_ERR_LAUNCH, "attention_decode_bulk: cannot reserve %d bytes of shared memory", bytes);
        configured = bytes;
    }
    const int work = p.n_rows * p.HKV * p.splits;
    int grid = CTAS * sm_count();
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    if (work < grid) grid = work;
    launch_overlapped(kernel, dim3(grid), dim3(BULK_THREADS), (size_t)bytes, stream, mkv, p);
    if (p.splits > 1)
        launch_overlapped(attention_combine_bulk_kernel<D>, dim3(p.n_rows, p.HQ), dim3(D < 128 ? D : 128), 0, stream,
                          (const float*)p.part_o, (const float*)p.part_ml, p.row_list, p.out, p.HQ, p.splits);
    return check_launch("attention_decode_bulk");
}

// Two CTAs per SM with three stages each when that fits the SM's shared memory, else two stages each, else one
// CTA with four stages: what counts is warps per SM (the consumers wait on dependent tensor-core instructions)
// and enough copies in flight.
template <int D> int launch_bulk(const CUtensorMap& mkv, const BulkParams& p, int max_ctas, cudaStream_t stream) {
    const int G = p.HQ / p.HKV;
    constexpr int SM_BYTES = 227 * 1024;
    const int b3 = bulk_smem_bytes(D, G, 3), b2 = bulk_smem_bytes(D, G, 2), b4 = bulk_smem_bytes(D, G, 4);
    if (2 * (b3 + 1024) <= SM_BYTES) return launch_config<D, 3, 2>(mkv, p, b3, max_ctas, stream);
    if (2 * (b2 + 1024) <= SM_BYTES) return launch_config<D, 2, 2>(mkv, p, b2, max_ctas, stream);
    return launch_config<D, 4, 1>(mkv, p, b4, max_ctas, stream);
}

}  // namespace

// num_pages: pages of the pool that k_base / v_base belong to (the copy engine needs the extent it may address).
PH_EXPORT int ph_attention_decode_bulk(const void* q, const void* k_base, const void* v_base, long long page_stride,
                                       int page_size, int num_pages, const int32_t* block_table, int table_stride,
                                       const int32_t* row_list, int n_rows, const int32_t* row_seg,
                                       const int32_t* positions, float* part_o, float* part_ml, void* out, int HQ,
                                       int HKV, int D, int splits, int window, float scale, int max_ctas,
                                       int* error_flag, cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !row_seg || !positions || !out || !error_flag || n_rows < 0 ||
        HQ < 1 || HKV < 1 || HQ % HKV || page_size < 1 || num_pages < 1 || window < 0 || splits < 1 ||
        (splits > 1 && (!part_o || !part_ml)))
        return fail(PH_ERR_ARG, "attention_decode_bulk: bad arguments (rows %d, HQ %d, HKV %d, splits %d)", n_rows, HQ, HKV, splits);
    if (D != 64 && D != 128) return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: head_dim %d is not 64 or 128", D);
    if (HQ / HKV > 16) return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: %d query heads per kv head exceed 16", HQ / HKV);
    if (page_size % 8 || BLOCK_KEYS % page_size)
        return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: pages of %d tokens (8, 16, 32 or 64 are taken)", page_size);
    if (page_stride % D || (((uintptr_t)q | (uintptr_t)k_base | (uintptr_t)v_base) & 15))
        return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: the cache is not laid out in whole, 16-byte aligned rows");
    if ((long long)n_rows * HKV * splits > 0x7fffffffLL) return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: too many work items");
    if (n_rows == 0) return PH_OK;
    // rows of the [rows, D] view that start at k_base (v_base) and stay inside the pool
    const long long rows_per_page = page_stride / D;
    const long long rows = (long long)(num_pages - 1) * rows_per_page + (long long)HKV * page_size;
    if (rows >= 0x7fffffffLL) return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: the pool has too many rows");
    const long long kv_stride_bytes = (const char*)v_base - (const char*)k_base;
    if (kv_stride_bytes <= 0 || kv_stride_bytes % 16)
        return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: values must follow keys at a multiple of 16 bytes");
    CUtensorMap mkv;
    if (!make_page_map(&mkv, k_base, kv_stride_bytes, rows, D, page_size))
        return fail(PH_ERR_UNSUPPORTED, "attention_decode_bulk: the copy engine does not take this cache layout "
                                        "(cuTensorMapEncodeTiled refused it)");
    BulkParams p;
    p.q = (const __nv_bfloat16*)q; p.rows_per_page = rows_per_page; p.total_rows = (int)rows;
    p.page_size = page_size; p.page_shift = page_size == 8 ? 3 : page_size == 16 ? 4 : page_size == 32 ? 5 : 6;
    p.block_table = block_table; p.table_stride = table_stride;
    p.row_list = row_list; p.row_seg = row_seg; p.positions = positions; p.part_o = part_o; p.part_ml = part_ml;
    p.out = (__nv_bfloat16*)out; p.n_rows = n_rows; p.HQ = HQ; p.HKV = HKV; p.splits = splits; p.window = window;
    p.scale_log2 = scale * LOG2E; p.error_flag = error_flag;
    return D == 64 ? launch_bulk<64>(mkv, p, max_ctas, stream) : launch_bulk<128>(mkv, p, max_ctas, stream);
}

// Prefill attention on the 5th-generation tensor cores (tcgen05), keys and values straight from cache pages.
//
// One CTA per (128 query tokens of one request, query head); two CTAs share an SM.  Roles inside a CTA:
//   warp 0    TMA producer: the query tile once (4-D box), then per block of 64 keys the pages' keys and values
//             (one box per page and 64-element half, 128-byte swizzled).  K and V have rings of their own: a K
//             tile is free once its S is done, a V tile once P V has read it.
//   warp 1    issues tcgen05.mma from one lane: S = Q K^T (M 128, N 64, K 128) into one of two score buffers in
//             tensor memory, and O += P V (M 128, N 128, K 64) with P read from tensor memory and V as an
//             MN-major operand from shared memory; O stays in tensor memory for the whole tile.  S of block b + 1
//             is issued before P V of block b, so the softmax never waits for its scores.
//   warps 2-5 softmax: thread i owns query row i.  It reads its row of S with tcgen05.ld (no shuffles: the row is
//             in one thread), masks only in blocks at the diagonal or the window's edge, keeps the running
//             maximum and sum in float32 (packed two-element float32 instructions, ex2.approx) and writes P as
//             bfloat16 pairs back over its scores with tcgen05.st.  The exponent's reference maximum only moves
//             when the row maximum has grown by more than 2^8 since it was set; then the row of O in tensor
//             memory is rescaled (tcgen05.ld / st).
// Tensor memory: columns 0-63 scores (then P) of even blocks, 64-191 O, 192-255 scores of odd blocks.
// A tile's keys may be shared by several CTAs (grid z), for a few tiles late in a long context: each leaves its
// unnormalised sums, its reference and its row sums in scratch, and a second kernel merges them.
// A row at absolute position z sees positions max(0, z - window + 1) .. z.  Pages past the tile's last token
// come from an out-of-range coordinate (zeros), scores of invisible keys are replaced by -inf and value rows
// after the last token inside its page are zeroed before P V, so unwritten page slots may hold anything.
// Every mbarrier wait is bounded and reports through an error word; TMEM is freed on every path.
// Math as in the reference's flash kernel: src/attention.hip:612-701; scale 1/sqrt(D): src/attention.cpp:197.
#include "common.cuh"
#include "mbarrier.cuh"

#include <cuda.h>
#include <math.h>

#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace ph;
namespace mb = ph_mbar;

constexpr int BM = 128;                 // query rows of a tile = M of the instruction
constexpr int BN = 64;                  // keys per block
constexpr int D = 128;                  // head size this kernel is built for
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr int HALF_Q = BM * 128;        // bytes of one 64-element half of the Q tile
constexpr int HALF_KV = BN * 128;       // bytes of one half of a K or V block
constexpr int Q_BYTES = 2 * HALF_Q;
constexpr int KV_BYTES = 2 * HALF_KV;   // K (or V) of one block
constexpr int TMEM_COLS = 256;          // S of even blocks: columns 0-63, O: 64-191, S of odd blocks: 192-255
constexpr int SMEM_BYTES = 1024 + Q_BYTES + KV_STAGES * 2 * KV_BYTES + 256;
constexpr float RESCALE_STEP = 8.0f;    // log2 units the row maximum may outgrow the reference before O is rescaled
constexpr float LOG2E = 1.4426950408889634f;

#define PH_ERR_WAIT_TC5_PRODUCER 121
#define PH_ERR_WAIT_TC5_MMA 122
#define PH_ERR_WAIT_TC5_SOFTMAX 123

struct Tc5Params {
    long long rows_per_page;
    int total_rows;
    int page_size, page_shift;
    const int32_t* block_table;
    int table_stride;
    const int32_t* seg_start;
    const int32_t* seg_ctx_len;
    const int32_t* tile_seg;
    const int32_t* tile_first;
    int n_tiles;
    __nv_bfloat16* out;
    int HQ, HKV, window;
    float scale_log2;
    int* error_flag;
    int splits;                    // CTAs that share a tile's keys (grid z); > 1: partial results, merged by a second kernel
    float* part_o;                 // [T][HQ][splits][D] unnormalised partial outputs
    float* part_ml;                // [T][HQ][splits][2] the exponent's reference and the sum of each partial
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptors, 128-byte swizzle, version 1 (bits 46-47), swizzle mode 2 (bits 61-63).
// K-major (rows of 128 bytes along K, groups of 8 rows sbo bytes apart) ignores the leading offset; MN-major
// (rows of 128 bytes = 64 elements along M or N, one row per k) uses it as the distance between 64-element
// chunks along M/N, and sbo as the distance between groups of 8 k.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D float32, A and B bfloat16, A K-major, B K-major (b_mn 0) or MN-major (1).
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// 2^x, one instruction; -inf gives 0.
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 operations in one instruction.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\n"
        "mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n.reg .b64 ra, rb, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
        "add.rn.f32x2 rd, ra, rb;\n"
        "mov.b64 {%0, %1}, rd;\n}"
        : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// A operand from tensor memory: 128 rows on the lanes, 16 bfloat16 of K in 8 columns.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const Tc5Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                   // [half][128 rows][128 B]
    unsigned char* k_ring = q_tile + Q_BYTES;                       // [stage][half][key][128 B]
    unsigned char* v_ring = k_ring + KV_STAGES * KV_BYTES;          // [stage][half][key][128 B]
    uint64_t* bars = (uint64_t*)(v_ring + KV_STAGES * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                  // [KV_STAGES] keys of a block have landed
    uint64_t* k_empty = k_full + KV_STAGES;       // [KV_STAGES] ... and the tile may be loaded again
    uint64_t* v_full = k_empty + KV_STAGES;       // [KV_STAGES] values of a block have landed
    uint64_t* v_empty = v_full + KV_STAGES;       // [KV_STAGES] ... and have been read
    uint64_t* s_full = v_empty + KV_STAGES;       // [2] S of a block is in tensor memory (two buffers in turn)
    uint64_t* p_full = s_full + 2;                // P of a block is written, O is rescaled
    uint64_t* o_full = p_full + 1;                // P V of a block has been added to O
    uint32_t* tmem_slot = (uint32_t*)(o_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the heads of one tile start together; the caller lists the tiles with the most keys first
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seg = p.tile_seg[tile], first = p.tile_first[tile];
    const int row0 = p.seg_start[seg], q_len = p.seg_start[seg + 1] - row0;
    const int ctx_len = p.seg_ctx_len[seg];
    const int n_rows = min(BM, q_len - first);
    const int z_first = ctx_len - q_len + first, z_last = z_first + n_rows - 1;
    const int lo_tile = p.window > 0 ? max(0, z_first - p.window + 1) : 0;
    const int lo_page = lo_tile - (lo_tile & (p.page_size - 1));
    const int tile_blocks = (z_last - lo_page) / BN + 1;          // blocks of 64 keys the tile sees
    // this CTA's share of them: blocks b_first .. b_first + n_blocks - 1 (none when the tile has fewer blocks than CTAs)
    const int per_split = (tile_blocks + p.splits - 1) / p.splits;
    const int b_first = (int)blockIdx.z * per_split;
    const int n_blocks = max(0, min(tile_blocks, b_first + per_split) - b_first);
    const int g = h / (p.HQ / p.HKV);

    if (threadIdx.x == 0) {
        mb::init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mb::init(&k_full[s], 1); mb::init(&k_empty[s], 1);
            mb::init(&v_full[s], 1); mb::init(&v_empty[s], 1);
        }
        mb::init(&s_full[0], 1);
        mb::init(&s_full[1], 1);
        mb::init(p_full, 4);
        mb::init(o_full, 1);
        mb::fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // only now, with this CTA's tensor memory in hand: a kernel started early beside it must not take the columns
    // this CTA still waits for while it waits for this kernel to end
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 64;
    auto tmem_s = [&](int b) { return tmem_base + ((b & 1) ? 192u : 0u); };
    // block b uses stage b % KV_STAGES for the (b / KV_STAGES)-th time
    auto stage_of = [](int b) { return b % KV_STAGES; };
    auto use_parity = [](int b) { return (uint32_t)((b / KV_STAGES) & 1); };

    if (warp == 0) {
        // ---- producer: K of block b, then V of block b - 1: the order in which their tiles come free ----
        const int32_t* table = p.block_table + (size_t)seg * p.table_stride;
        const int psh = p.page_shift, ppb = BN >> psh;
        int ok = 1;
        if (lane == 0 && n_blocks > 0) {
            mb::arrive_expect_tx(q_full, Q_BYTES);
            tma_load_4d(q_tile, &map_q, q_full, 0, row0 + first, 0, h);       // box {64, 128 rows, 2 halves, 1 head}
        }
        auto load = [&](int b, bool is_v) {
            const int stage = stage_of(b);
            uint64_t* full = is_v ? &v_full[stage] : &k_full[stage];
            if (lane == 0) {
                ok = mb::wait(is_v ? &v_empty[stage] : &k_empty[stage], use_parity(b) ^ 1, p.error_flag, PH_ERR_WAIT_TC5_PRODUCER) ? 1 : 0;
                if (ok) mb::arrive_expect_tx(full, KV_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) return;
            // lane (page j, half) issues one box
            if (lane < ppb * 2) {
                const int pj = lane >> 1, half = lane & 1;
                const int pos = lo_page + (b_first + b) * BN + (pj << psh);
                int row = p.total_rows;                       // past the tile's last token: zeros
                if (pos <= z_last) row = (int)((long long)table[pos >> psh] * p.rows_per_page + (long long)g * p.page_size);
                unsigned char* dst = (is_v ? v_ring : k_ring) + stage * KV_BYTES + half * HALF_KV + (pj << psh) * 128;
                tma_load_2d(dst, is_v ? &map_v : &map_k, full, half * 64, row);
            }
        };
        for (int b = 0; b <= n_blocks && ok; ++b) {
            if (b < n_blocks) load(b, false);
            if (b > 0 && ok) load(b - 1, true);
        }
        if (lane == 0 && ok) {
            // no copy may be in flight when the CTA ends: the last blocks' tiles have been read
            for (int b = max(0, n_blocks - KV_STAGES); b < n_blocks; ++b) {
                if (!mb::wait(&k_empty[stage_of(b)], use_parity(b), p.error_flag, PH_ERR_WAIT_TC5_PRODUCER)) break;
                if (!mb::wait(&v_empty[stage_of(b)], use_parity(b), p.error_flag, PH_ERR_WAIT_TC5_PRODUCER)) break;
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issue ----
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(BM, BN, 0);      // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = make_idesc(BM, D, 1);       // O += P V: V is MN-major
            bool ok = n_blocks == 0 || mb::wait(q_full, 0, p.error_flag, PH_ERR_WAIT_TC5_MMA);
            // S of block b + 1 is issued before P V of block b where its keys have landed, so that the softmax of
            // the next block finds its scores ready while the tensor core adds this block to O.  Its buffer in
            // tensor memory held S (and P) of block b - 1, whose P V was issued before: the pipe keeps the order.
            auto issue_s = [&](int b) {
                const uint32_t k_tile = smem_u32(k_ring + stage_of(b) * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * HALF_Q + (ks & 3) * 32, offk = (ks >> 2) * HALF_KV + (ks & 3) * 32;
                    umma_bf16(tmem_s(b), make_desc(smem_u32(q_tile) + off, 16, 1024), make_desc(k_tile + offk, 16, 1024), idesc_s,
                              ks > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[b & 1]);
                umma_commit(&k_empty[stage_of(b)]);      // the keys are not needed again
            };
            if (ok && n_blocks > 0) {
                ok = mb::wait(&k_full[0], 0, p.error_flag, PH_ERR_WAIT_TC5_MMA);
                if (ok) { tc_fence_after(); issue_s(0); }
            }
            for (int b = 0; b < n_blocks && ok; ++b) {
                const int stage = stage_of(b);
                bool next_issued = b + 1 >= n_blocks;
                if (!next_issued && mb::test_wait(&k_full[stage_of(b + 1)], use_parity(b + 1))) {
                    tc_fence_after();
                    issue_s(b + 1);
                    next_issued = true;
                }
                if (!mb::wait(p_full, b & 1, p.error_flag, PH_ERR_WAIT_TC5_MMA)) { ok = false; break; }
                if (!mb::wait(&v_full[stage], use_parity(b), p.error_flag, PH_ERR_WAIT_TC5_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_tile = smem_u32(v_ring + stage * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // A: 16 keys = 8 columns further in tensor memory; B: 16 keys = two groups of 8 rows further down V
                    umma_bf16_ts(tmem_o, tmem_s(b) + ks * 8, make_desc(v_tile + ks * 2048, HALF_KV, 1024), idesc_o,
                                 (b > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(o_full);
                umma_commit(&v_empty[stage]);
                if (!next_issued) {
                    if (!mb::wait(&k_full[stage_of(b + 1)], use_parity(b + 1), p.error_flag, PH_ERR_WAIT_TC5_MMA)) { ok = false; break; }
                    tc_fence_after();
                    issue_s(b + 1);
                }
            }
        }
    } else {
        // ---- softmax: thread = query row ----
        const int q = warp & 3;                          // TMEM lane quarter of this warp
        const int r = q * 32 + lane;                     // row of the tile
        const int z = z_first + min(r, n_rows - 1);      // rows past the portion repeat the last one; never stored
        const int lo = p.window > 0 ? max(0, z - p.window + 1) : 0;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        float m_ref = -INFINITY;                         // the maximum the exponents refer to
        float l = 0.0f;
        bool ok = true;
        for (int b = 0; b < n_blocks && ok; ++b) {
            const int key0 = lo_page + (b_first + b) * BN;
            const int stage = stage_of(b);
            if (!mb::wait(&s_full[b & 1], (b >> 1) & 1, p.error_flag, PH_ERR_WAIT_TC5_SOFTMAX)) { ok = false; break; }
            tc_fence_after();
            // the row's 64 scores, as pairs
            float2 s[BN / 2];
            {
                uint32_t raw[BN];
                tmem_ld32(tmem_s(b) + lane_addr, raw);
                tmem_ld32(tmem_s(b) + lane_addr + 32, raw + 32);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < BN / 2; ++j) s[j] = make_float2(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1]));
            }
            if (key0 + BN - 1 > z || key0 < lo) {            // only the blocks at the diagonal and at the window's edge
#pragma unroll
                for (int j = 0; j < BN / 2; ++j) {
                    if (key0 + 2 * j > z || key0 + 2 * j < lo) s[j].x = -INFINITY;
                    if (key0 + 2 * j + 1 > z || key0 + 2 * j + 1 < lo) s[j].y = -INFINITY;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < BN / 2; j += 2) {
                mx0 = fmaxf(mx0, fmaxf(s[j].x, s[j].y));
                mx1 = fmaxf(mx1, fmaxf(s[j + 1].x, s[j + 1].y));
            }
            const float mx = fmaxf(mx0, mx1) * p.scale_log2;       // the scale is positive: the maximum commutes with it
            // move the reference only when the maximum has outgrown it by more than RESCALE_STEP
            float corr = 1.0f;
            if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY)) {
                corr = ex2(m_ref - mx);                   // 0 the first time
                m_ref = mx;
            }
            // P = 2^(s * scale - reference) as bfloat16 pairs over the first 32 columns of this block's scores
            const float neg_ref = m_ref == -INFINITY ? 0.0f : -m_ref;
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg2 = make_float2(neg_ref, neg_ref);
            float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
            uint32_t packed[BN / 2];
#pragma unroll
            for (int j = 0; j < BN / 2; j += 2) {
                const float2 a0 = fma2(s[j], scale2, neg2), a1 = fma2(s[j + 1], scale2, neg2);
                const float2 e0 = make_float2(ex2(a0.x), ex2(a0.y)), e1 = make_float2(ex2(a1.x), ex2(a1.y));
                sum_a = add2(sum_a, e0);
                sum_b = add2(sum_b, e1);
                __nv_bfloat162 h0 = __floats2bfloat162_rn(e0.x, e0.y), h1 = __floats2bfloat162_rn(e1.x, e1.y);
                packed[j] = *(uint32_t*)&h0;
                packed[j + 1] = *(uint32_t*)&h1;
            }
            tmem_st32(tmem_s(b) + lane_addr, packed);
            const float sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
            l = l * corr + sum;
            // O of the blocks so far must be complete before it is rescaled, and before P V of this block is issued
            if (b > 0) {
                if (!mb::wait(o_full, (b - 1) & 1, p.error_flag, PH_ERR_WAIT_TC5_SOFTMAX)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t raw[32];
                        tmem_ld32(tmem_o + lane_addr + c * 32, raw);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(__uint_as_float(raw[j]) * corr);
                        tmem_st32(tmem_o + lane_addr + c * 32, raw);
                    }
                }
            }
            if (b_first + b == tile_blocks - 1) {
                // value rows after the tile's last token inside its page may hold anything: zero them
                if (!mb::wait(&v_full[stage], use_parity(b), p.error_flag, PH_ERR_WAIT_TC5_SOFTMAX)) { ok = false; break; }
                unsigned char* v_tile = v_ring + stage * KV_BYTES;
                const int first_bad = z_last - key0 + 1;
                for (int idx = r; idx < (BN - first_bad) * 16; idx += 128) {
                    const int row = first_bad + idx / 16, c = idx % 16;
                    *(uint4*)(v_tile + (c >> 3) * HALF_KV + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zeros, before the tensor core reads them
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mb::arrive(p_full);
        }
        if (ok && n_blocks > 0) ok = mb::wait(o_full, (n_blocks - 1) & 1, p.error_flag, PH_ERR_WAIT_TC5_SOFTMAX);
        if (ok && p.splits == 1) {
            tc_fence_after();
            const float inv = l == 0.0f ? 0.0f : 1.0f / l;        // a row with no visible key gives 0; NaN stays NaN
            __nv_bfloat16* dst = p.out + (size_t)(row0 + first + r) * p.HQ * D + (size_t)h * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t raw[32];
                tmem_ld32(tmem_o + lane_addr + c * 32, raw);          // warp-wide: every lane takes part
                tmem_ld_wait();
                if (r < n_rows) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(raw[j]) * inv, __uint_as_float(raw[j + 1]) * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(raw[j + 2]) * inv, __uint_as_float(raw[j + 3]) * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(raw[j + 4]) * inv, __uint_as_float(raw[j + 5]) * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(raw[j + 6]) * inv, __uint_as_float(raw[j + 7]) * inv);
                        uint4 v;
                        v.x = *(uint32_t*)&h0; v.y = *(uint32_t*)&h1; v.z = *(uint32_t*)&h2; v.w = *(uint32_t*)&h3;
                        *(uint4*)(dst + c * 32 + j) = v;
                    }
                }
            }
        } else if (ok) {
            // one of several CTAs on this tile: the unnormalised sums, their reference and the row sums go to scratch
            tc_fence_after();
            const size_t slot = ((size_t)(row0 + first + r) * p.HQ + h) * p.splits + blockIdx.z;
            if (r < n_rows) {
                p.part_ml[slot * 2] = m_ref;                          // -inf, with a sum of 0, when this CTA saw no key of the row
                p.part_ml[slot * 2 + 1] = l;
            }
            if (n_blocks > 0) {
                float* dst = p.part_o + slot * D;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t raw[32];
                    tmem_ld32(tmem_o + lane_addr + c * 32, raw);
                    tmem_ld_wait();
                    if (r < n_rows) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) *(uint4*)(dst + c * 32 + j) = make_uint4(raw[j], raw[j + 1], raw[j + 2], raw[j + 3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Merges the partial results of the CTAs that shared a tile's keys: grid (tile, head, groups of four rows), a warp per
// row, four dimensions per lane, every partial of the row fetched before any is used.  A partial with reference -inf
// saw no key of the row and is skipped (its output slot was never written).
constexpr int MERGE_MAX = 16;      // most CTAs per tile
__global__ void __launch_bounds__(128)
attention_prefill_tc5_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     const int32_t* __restrict__ seg_start, const int32_t* __restrict__ tile_seg,
                                     const int32_t* __restrict__ tile_first, __nv_bfloat16* __restrict__ out, int HQ, int splits) {
    pdl_launch_dependents();
    const int tile = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = tile_seg[tile], first = tile_first[tile];
    const int row0 = seg_start[seg], n_rows = min(BM, seg_start[seg + 1] - row0 - first);
    const int r = blockIdx.z * 4 + warp;
    pdl_wait();
    if (r >= n_rows) return;
    const size_t slot0 = ((size_t)(row0 + first + r) * HQ + h) * splits;
    float ms[MERGE_MAX], ls[MERGE_MAX];
    float4 o[MERGE_MAX];
    float m = -INFINITY;
#pragma unroll
    for (int s = 0; s < MERGE_MAX; ++s) {
        ms[s] = s < splits ? part_ml[(slot0 + s) * 2] : -INFINITY;
        ls[s] = s < splits ? part_ml[(slot0 + s) * 2 + 1] : 0.0f;
        m = fmaxf(m, ms[s]);
    }
#pragma unroll
    for (int s = 0; s < MERGE_MAX; ++s)
        o[s] = s < splits && ms[s] != -INFINITY ? *(const float4*)(part_o + (slot0 + s) * D + lane * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float l = 0.0f;
#pragma unroll
    for (int s = 0; s < MERGE_MAX; ++s) {
        if (ms[s] == -INFINITY) continue;
        const float c = exp2f(ms[s] - m);
        acc.x += c * o[s].x; acc.y += c * o[s].y; acc.z += c * o[s].z; acc.w += c * o[s].w;
        l += c * ls[s];
    }
    const float inv = l == 0.0f ? 0.0f : 1.0f / l;        // a row with no visible key gives 0; NaN stays NaN
    __nv_bfloat162 h0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), h1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 v;
    v.x = *(uint32_t*)&h0; v.y = *(uint32_t*)&h1;
    *(uint2*)(out + ((size_t)(row0 + first + r) * HQ + h) * D + lane * 4) = v;
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

bool encode(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, cuuint64_t, cuuint64_t, cuuint64_t, cuuint32_t>, CUtensorMap> cache;
    const auto key = std::make_tuple(base, rank, dims[1], strides[0], rank > 3 ? dims[3] : 0, box[1]);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
}

}  // namespace

PH_DEFINE_LAST_ERROR(ph_flash5)

// q [T, HQ, 128] bfloat16 -> out [T, HQ * 128].  splits > 1: that many CTAs share the keys of every tile and leave
// partial results in part_o [T][HQ][splits][128] and part_ml [T][HQ][splits][2] (float32), which a second kernel merges;
// for few tiles that look far back.  tile_seg / tile_first: the step's prompt portions cut into tiles
// of 128 rows (segment, first row of the tile within the portion).  num_pages: pages of the pool that k_base /
// v_base belong to.
PH_EXPORT int ph_attention_prefill_tc5(const void* q, int T, const void* k_base, const void* v_base, long long page_stride,
                                       int page_size, int num_pages, const int32_t* block_table, int table_stride,
                                       const int32_t* seg_start, const int32_t* seg_ctx_len, const int32_t* tile_seg,
                                       const int32_t* tile_first, int n_tiles, void* out, int HQ, int HKV, int head_dim,
                                       int window, float scale, int splits, float* part_o, float* part_ml,
                                       int* error_flag, cudaStream_t stream) {
    if (!q || !k_base || !v_base || !block_table || !seg_start || !seg_ctx_len || !tile_seg || !tile_first || !out ||
        !error_flag || T < 1 || n_tiles < 0 || HQ < 1 || HKV < 1 || HQ % HKV || num_pages < 1 || window < 0 || !(scale > 0.0f))
        return fail(PH_ERR_ARG, "attention_prefill_tc5: bad arguments (tiles %d, HQ %d, HKV %d)", n_tiles, HQ, HKV);
    if (head_dim != D) return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: head_dim %d is not %d", head_dim, D);
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)
        return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: pages of %d tokens (8, 16, 32 or 64 are taken)", page_size);
    if (page_stride % D || (((uintptr_t)q | (uintptr_t)k_base | (uintptr_t)v_base | (uintptr_t)out) & 15))
        return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: tensors must be 16-byte aligned, pages whole rows");
    if (n_tiles > 65535) return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: %d tiles exceed the grid", n_tiles);
    if (splits < 1 || splits > MERGE_MAX || (splits > 1 && (!part_o || !part_ml || (((uintptr_t)part_o) & 15))))
        return fail(PH_ERR_ARG, "attention_prefill_tc5: %d splits need 16-byte aligned scratch for the partial results", splits);
    if (n_tiles == 0) return PH_OK;
    const long long rows_per_page = page_stride / D;
    const long long rows = (long long)(num_pages - 1) * rows_per_page + (long long)HKV * page_size;
    if (rows >= 0x7fffffffLL) return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: the pool has too many rows");
    CUtensorMap mq, mk, mv;
    // Q: {64 elements, T tokens (HQ * D * 2 bytes apart), 2 halves (128 bytes apart), HQ heads (D * 2 bytes apart)}
    const cuuint64_t qdims[4] = {64, (cuuint64_t)T, 2, (cuuint64_t)HQ};
    const cuuint64_t qstrides[3] = {(cuuint64_t)HQ * D * 2, 128, (cuuint64_t)D * 2};
    const cuuint32_t qbox[4] = {64, BM, 2, 1};
    // K, V: [rows, D] from the entry's first element; a box is one 64-element half of one page of one kv head
    const cuuint64_t kdims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    const cuuint64_t kstrides[1] = {(cuuint64_t)D * 2};
    const cuuint32_t kbox[2] = {64, (cuuint32_t)page_size};
    if (!encode(&mq, q, 4, qdims, qstrides, qbox) || !encode(&mk, k_base, 2, kdims, kstrides, kbox) ||
        !encode(&mv, v_base, 2, kdims, kstrides, kbox))
        return fail(PH_ERR_UNSUPPORTED, "attention_prefill_tc5: cuTensorMapEncodeTiled refused the layout");
    Tc5Params p;
    p.rows_per_page = rows_per_page; p.total_rows = (int)rows; p.page_size = page_size; p.page_shift = page_size == 8 ? 3 : page_size == 16 ? 4 : page_size == 32 ? 5 : 6;
    p.block_table = block_table; p.table_stride = table_stride; p.seg_start = seg_start; p.seg_ctx_len = seg_ctx_len;
    p.tile_seg = tile_seg; p.tile_first = tile_first; p.n_tiles = n_tiles; p.out = (__nv_bfloat16*)out;
    p.HQ = HQ; p.HKV = HKV; p.window = window; p.scale_log2 = scale * LOG2E; p.error_flag = error_flag;
    p.splits = splits; p.part_o = part_o; p.part_ml = part_ml;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return fail(PH_ERR_LAUNCH, "attention_prefill_tc5: cannot reserve %d bytes of shared memory", SMEM_BYTES);
        configured = true;
    }
    launch_overlapped(attention_prefill_tc5_kernel, dim3(HQ, n_tiles, splits), dim3(THREADS), (size_t)SMEM_BYTES, stream, mq, mk, mv, p);
    if (splits > 1)
        launch_overlapped(attention_prefill_tc5_combine_kernel, dim3(n_tiles, HQ, BM / 4), dim3(128), 0, stream,
                          (const float*)part_o, (const float*)part_ml, seg_start, tile_seg, tile_first, (__nv_bfloat16*)out, HQ, splits);
    return check_launch("attention_prefill_tc5");
}

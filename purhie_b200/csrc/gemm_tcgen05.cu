// bfloat16 matrix product on the 5th-generation tensor cores: D[a, b] = sum_k A[a, k] * B[b, k], both
// operands K-major in global memory, float32 accumulation in tensor memory (TMEM).
//
// One persistent CTA per SM walks over work items (tile of 128 A-rows x BN B-rows, split of K).  Warp 0 is
// the TMA producer (one elected lane): it copies 128 x 64 and BN x 64 element boxes, 128-byte swizzled, into
// a ring of shared-memory stages and signals a "full" mbarrier per stage.  Warp 1 allocates TMEM and issues
// tcgen05.mma (M = 128, N = BN, K = 16 per instruction) from one lane, releasing a stage with
// tcgen05.commit.  Warps 2-5 are the epilogue: they read the accumulator with tcgen05.ld (each warp its own
// 32-lane quarter), convert and store it, while the MMA warp already fills the second accumulator buffer.
//
// Two orientations share the kernel.  Plain: A = activations [tokens, K], B = weight [features, K], the
// thread that holds accumulator row a writes out[a, b0 .. b0+BN).  Swapped (few tokens: decoding): A =
// weight, B = activations, so that the 128-row side of the instruction is filled by output features and the
// few tokens sit on the N side; the accumulator is stored transposed, out[b, a].  With splits > 1 each
// split of K writes its own float32 partial result [split][tokens][features]; whoever consumes the product
// adds the partials in order (the norm, rotary and activation kernels take them), which keeps the sum
// deterministic.
//
// No cluster multicast is used: every CTA fetches its own tiles.  Every wait on an mbarrier is bounded; a
// wait that runs out sets *error_flag, and the CTA still frees its TMEM and returns.
// The reference's counterpart is its WMMA tile kernel for gfx1151 (src/matvec_q.hip:3437-3547).
#include "common.cuh"

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace ph;

constexpr int BM = 128;          // rows of the A tile = M of the instruction
constexpr int BK = 64;           // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

#define PH_ERR_WAIT_PRODUCER 101
#define PH_ERR_WAIT_MMA 102
#define PH_ERR_WAIT_EPILOGUE 103

struct GemmParams {
    int rows_a, rows_b, K;
    int a_tiles, b_tiles, splits, kblocks;
    void* out;
    int out_bf16;        // 1: bfloat16 output, 0: float32
    int swapped;
    int accumulate;      // 1: out (float32, plain orientation, one split) += the product: the residual sum in the epilogue
    int swiglu;          // 1: columns are (gate, up) pairs; out[a, j] = silu(D[a, 2j]) * D[a, 2j + 1] (plain orientation)
    long long ld;        // row length of out
    long long split_stride;
    // A factor per token that the norm in front left out of the activations, rsqrt(sum over the chunks of
    // row_sumsq[token][chunk] / row_width + row_eps), applied to the accumulator before anything else happens to it
    // (the product is linear in its rows).  Swapped orientation: bfloat16 output; plain orientation: tiles of 256
    // columns, one split, no accumulate.  Null: none.
    const float* row_sumsq;
    int row_chunks, row_width;
    float row_eps;
    // Plain orientation with accumulate, tiles of 256 columns: what the norm after this addition would do is done here.
    // Beside out += product, the new rows times norm_weight go to norm_rows (bfloat16, [rows_a, ld]) and each row's sum
    // of squares over 128 columns to norm_sumsq[row][column / 128] ([rows_a, 2 * b_tiles]): the rows lack the factor
    // rsqrt(sum over the entries / ld + eps), which their consumer applies (row_sumsq above).  Null: none.
    const float* norm_weight;
    __nv_bfloat16* norm_rows;
    float* norm_sumsq;
    // Pair kernel, results that are stored, not added: the epilogue leaves boxes of 32 rows x 128 bytes in shared memory
    // and the copy engine stores them (whole lines, nothing for the warps to wait for).  1: bfloat16 output of whole
    // sums (plain or with the activation), boxes of 64 columns; 2: float32 (whole or partial sums), boxes of 32 columns
    // of out seen as [splits][rows][columns].  0: the warps store.
    int tma_store;
    int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false (after setting the error flag) when the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && global_timer() - t0 > WAIT_LIMIT_NS) {
            atomicExch(error_flag, code);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c_inner, int c_row) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c_inner), "r"(c_row) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups of 8
// rows 1024 bytes apart.  Bits: [0,14) address >> 4, [16,30) leading byte offset >> 4 (unused with this
// swizzle), [32,46) stride byte offset >> 4, [46,48) version 1, [61,64) swizzle mode 2 (128 bytes).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: D float32 (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1), both
// K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Few tokens (BN <= 64: weight streaming): two CTAs share an SM, each with half the stages, so that one CTA's
// start-up and epilogue overlap the other's streaming.  Many tokens: one CTA per SM with all the stages.
template <int BN> struct TileConfig {
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int CTAS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int BUDGET = (CTAS_PER_SM == 2 ? 104 : 200) * 1024;
    static constexpr int STAGES = (BUDGET / STAGE_BYTES) > 10 ? 10 : (BUDGET / STAGE_BYTES);
    static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : 2 * BN;          // a power of two: BN is one
    // per epilogue warp: 32 tokens x 32 features in bfloat16 (swapped), 32 rows x 32 columns in float32 (plain, tiles of 256)
    static constexpr int STAGING_BYTES = 4 * 32 * 32 * (BN == 256 ? 4 : 2);
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */ + STAGING_BYTES;
};

// Plain orientation: the factor that the norm in front left out of row a of the activations.
__device__ __forceinline__ float plain_row_factor(const GemmParams& p, int a) {
    if (a >= p.rows_a) return 1.0f;
    float s = 0.0f;
    for (int k = 0; k < p.row_chunks; ++k) s += p.row_sumsq[(size_t)a * p.row_chunks + k];
    return rsqrtf(s / (float)p.row_width + p.row_eps);
}

// One chunk of CH accumulator columns of row a, starting at column b0 + c of the tile, to its place in out.
template <int CH>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const uint32_t* r, int a, int b0, int c, size_t split_off) {
    if (a >= p.rows_a) return;
    if (p.swiglu) {
        // the activation in the epilogue: the product itself never goes to memory
        const size_t base = (size_t)a * p.ld + (size_t)((b0 + c) >> 1);
        float h[CH / 2];
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) {
            const float g = __uint_as_float(r[2 * j]), u = __uint_as_float(r[2 * j + 1]);
            h[j] = g / (1.0f + __expf(-g)) * u;
        }
        const bool full_chunk = (b0 + c + CH <= p.rows_b);
        if (p.out_bf16) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + base;
            if (full_chunk && ((uintptr_t)o & 15) == 0) {
#pragma unroll
                for (int j = 0; j < CH / 2; j += 8) {
                    uint4 v;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(h[j], h[j + 1]), h1 = __floats2bfloat162_rn(h[j + 2], h[j + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(h[j + 4], h[j + 5]), h3 = __floats2bfloat162_rn(h[j + 6], h[j + 7]);
                    v.x = *(uint32_t*)&h0; v.y = *(uint32_t*)&h1; v.z = *(uint32_t*)&h2; v.w = *(uint32_t*)&h3;
                    *(uint4*)(o + j) = v;
                }
            } else {
#pragma unroll
                for (int j = 0; j < CH / 2; ++j)
                    if (b0 + c + 2 * j + 1 < p.rows_b) o[j] = __float2bfloat16_rn(h[j]);
            }
        } else {
            float* o = (float*)p.out + base;
#pragma unroll
            for (int j = 0; j < CH / 2; ++j)
                if (b0 + c + 2 * j + 1 < p.rows_b) o[j] = h[j];
        }
    } else if (!p.swapped) {
        const size_t base = split_off + (size_t)a * p.ld + (size_t)(b0 + c);
        const bool full_chunk = (b0 + c + CH <= p.rows_b);
        if (p.out_bf16) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + base;
            if (full_chunk && ((uintptr_t)o & 15) == 0) {
#pragma unroll
                for (int j = 0; j < CH; j += 8) {
                    uint4 v;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                    v.x = *(uint32_t*)&h0; v.y = *(uint32_t*)&h1; v.z = *(uint32_t*)&h2; v.w = *(uint32_t*)&h3;
                    *(uint4*)(o + j) = v;
                }
            } else {
#pragma unroll
                for (int j = 0; j < CH; ++j)
                    if (b0 + c + j < p.rows_b) o[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
        } else {
            float* o = (float*)p.out + base;
            if (full_chunk && ((uintptr_t)o & 15) == 0) {
                if (p.accumulate) {
                    float4 old[CH / 4];
#pragma unroll
                    for (int j = 0; j < CH; j += 4) old[j / 4] = *(const float4*)(o + j);
#pragma unroll
                    for (int j = 0; j < CH; j += 4)
                        *(float4*)(o + j) = make_float4(old[j / 4].x + __uint_as_float(r[j]), old[j / 4].y + __uint_as_float(r[j + 1]),
                                                        old[j / 4].z + __uint_as_float(r[j + 2]), old[j / 4].w + __uint_as_float(r[j + 3]));
                } else {
#pragma unroll
                    for (int j = 0; j < CH; j += 4)
                        *(uint4*)(o + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CH; ++j)
                    if (b0 + c + j < p.rows_b) o[j] = p.accumulate ? o[j] + __uint_as_float(r[j]) : __uint_as_float(r[j]);
            }
        }
    } else {
        // transposed: this thread's accumulator row is output feature a; lanes are neighbours in a
        if (p.out_bf16) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + split_off + a;
#pragma unroll
            for (int j = 0; j < CH; ++j)
                if (b0 + c + j < p.rows_b) o[(size_t)(b0 + c + j) * p.ld] = __float2bfloat16_rn(__uint_as_float(r[j]));
        } else {
            float* o = (float*)p.out + split_off + a;
#pragma unroll
            for (int j = 0; j < CH; ++j)
                if (b0 + c + j < p.rows_b) o[(size_t)(b0 + c + j) * p.ld] = __uint_as_float(r[j]);
        }
    }
}

// Plain orientation, tiles of 256 columns, out += product: 32 columns of the warp's 32 rows pass through the warp's
// staging buffer (float32 [32][32], 16-byte slots swizzled by the row), so that lanes 8k .. 8k + 7 take row
// 4 it + k, four columns each, and the values that are added to can be asked for a chunk ahead, row by row, while the
// chunk before is still being worked on (a thread that walked along its own accumulator row would wait for its loads
// once per chunk, with nothing else to do).
// Vector form: every lane's four columns exist and are 16-byte aligned; else element by element, without the load ahead.
__device__ __forceinline__ bool accumulate_in_vectors(const GemmParams& p) {
    return (p.ld & 3) == 0 && ((uintptr_t)p.out & 15) == 0 && (p.rows_b & 3) == 0;
}
// The values of out that chunk c of the warp's rows is added to (zeros outside of out).
__device__ __forceinline__ void load_accumulate_chunk(const GemmParams& p, int row0, int lane, int b0, int c, float4* old) {
    const int col = b0 + c + (lane & 7) * 4;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int a = row0 + it * 4 + (lane >> 3);
        old[it] = (a < p.rows_a && col < p.rows_b) ? *(const float4*)((const float*)p.out + (size_t)a * p.ld + (size_t)col)
                                                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
}
// r: this lane's accumulator row; old: what load_accumulate_chunk fetched for this chunk (vector form only).
// With the norm ahead, the new rows times the norm's weight go to norm_rows, and ss[it] gathers this lane's share of
// the sum of squares of row 4 it + lane / 8.  Every lane of the warp calls this.
// next_c >= 0 (vector form): once the accumulator chunk is in shared memory and its registers are free, the values
// that chunk next_c is added to are asked for, into old_next.
__device__ __forceinline__ void store_chunk_accumulate_staged(const GemmParams& p, const uint32_t* r, const float4* old, bool vectors,
                                                              float* buf, int row0, int lane, int b0, int c, float* ss,
                                                              float4* old_next, int next_c) {
    float4* mine = (float4*)(buf + lane * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j)
        mine[j ^ (lane & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                           __uint_as_float(r[4 * j + 3]));
    __syncwarp();
    if (vectors && next_c >= 0) load_accumulate_chunk(p, row0, lane, b0, next_c, old_next);
    const int sub = lane >> 3, slot = lane & 7;
    const int col = b0 + c + slot * 4;                               // first of this lane's four columns
    const bool ahead = p.norm_weight != nullptr;
    float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (ahead && vectors && col < p.rows_b) g = __ldg((const float4*)(p.norm_weight + col));
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int rr = it * 4 + sub, a = row0 + rr;
        float4 v = ((const float4*)(buf + rr * 32))[slot ^ (rr & 7)];
        if (a >= p.rows_a || col >= p.rows_b) continue;
        const size_t at = (size_t)a * p.ld + (size_t)col;
        float* o = (float*)p.out + at;
        if (vectors) {
            v = make_float4(old[it].x + v.x, old[it].y + v.y, old[it].z + v.z, old[it].w + v.w);
            *(float4*)o = v;
            if (ahead) {
                ss[it] += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * g.x, v.y * g.y), hi = __floats2bfloat162_rn(v.z * g.z, v.w * g.w);
                *(uint2*)(p.norm_rows + at) = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);   // ld % 4 == 0: 8-byte aligned
            }
        } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (col + k < p.rows_b) {
                    const float x = o[k] + e[k];
                    o[k] = x;
                    if (ahead) {
                        ss[it] += x * x;
                        p.norm_rows[at + k] = __float2bfloat16_rn(x * __ldg(p.norm_weight + col + k));
                    }
                }
        }
    }
    __syncwarp();                                                    // the buffer is written again for the next chunk
}

// The sums of squares of the warp's rows over 128 columns (half of a tile's), to norm_sumsq[row][half_index]; a row has
// two entries per tile.
__device__ __forceinline__ void store_tile_sumsq(const GemmParams& p, float* ss, int row0, int lane, int half_index) {
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        float s = ss[it];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        const int a = row0 + it * 4 + (lane >> 3);
        if ((lane & 7) == 0 && a < p.rows_a) p.norm_sumsq[(size_t)a * (2 * p.b_tiles) + half_index] = s;
        ss[it] = 0.0f;
    }
}

// Swapped orientation with the activation: accumulator row a is output feature a, and gate and up features are
// neighbours (rows 2i and 2i + 1), so neighbouring lanes hold a pair; the even lane writes out[token, a / 2].
// Every lane of the warp calls this (the exchange needs them all).
template <int CH>
__device__ __forceinline__ void store_chunk_swapped_swiglu(const GemmParams& p, const uint32_t* r, int a, int b0, int c) {
    const bool writer = (a & 1) == 0 && a + 1 < p.rows_a;
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const float mine = __uint_as_float(r[j]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
        if (writer && b0 + c + j < p.rows_b) {
            const float h = mine / (1.0f + __expf(-mine)) * other;
            const size_t at = (size_t)(b0 + c + j) * p.ld + (size_t)(a >> 1);
            if (p.out_bf16) ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(h);
            else ((float*)p.out)[at] = h;
        }
    }
}

// Swapped orientation, bfloat16 output (plain or with the activation): the warp's 32 features x CH tokens go through
// its own staging buffer in shared memory, [token][feature], and leave as 16-byte vectors along the features
// instead of one 2-byte store per value.  With the activation, gate and up features are neighbouring lanes: the
// even lane works out token j, the odd lane token j + 1 of every pair of tokens, after one exchange.
// a_base: the warp's first output feature; every lane of the warp calls this.
// factor: lane (c + l) % 32 holds the factor of token b0 + c + l (1 where the norm left none out).
template <int CH>
__device__ __forceinline__ void store_chunk_swapped_bf16(const GemmParams& p, uint32_t* r, __nv_bfloat16* buf, int a_base,
                                                         int lane, int b0, int c, float factor) {
    const int W = p.swiglu ? 16 : 32;                 // output columns of this warp
    if (p.row_sumsq) {
#pragma unroll
        for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * __shfl_sync(0xffffffffu, factor, (c + j) & 31));
    }
    if (p.swiglu) {
        const int odd = lane & 1;
#pragma unroll
        for (int j = 0; j < CH; j += 2) {
            const float m0 = __uint_as_float(r[j]), m1 = __uint_as_float(r[j + 1]);
            const float got = __shfl_xor_sync(0xffffffffu, odd ? m0 : m1, 1);
            const float gate = odd ? got : m0, up = odd ? m1 : got;
            buf[(j + odd) * 16 + (lane >> 1)] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
        }
    } else {
#pragma unroll
        for (int j = 0; j < CH; ++j) buf[j * 32 + lane] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
    __syncwarp();
    const int vec_per_row = W / 8;
    const int first = p.swiglu ? a_base / 2 : a_base, limit = p.swiglu ? p.rows_a / 2 : p.rows_a;
    for (int idx = lane; idx < CH * vec_per_row; idx += 32) {
        const int row = idx / vec_per_row, v = idx % vec_per_row;
        const int token = b0 + c + row, col = first + v * 8;
        if (token >= p.rows_b || col >= limit) continue;
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)token * p.ld + col;
        const __nv_bfloat16* src = buf + row * W + v * 8;
        if (col + 8 <= limit && ((uintptr_t)dst & 15) == 0) {
            *(uint4*)dst = *(const uint4*)src;
        } else {
            for (int e = 0; e < 8 && col + e < limit; ++e) dst[e] = src[e];
        }
    }
    __syncwarp();                                      // the buffer is written again for the next chunk
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, TileConfig<BN>::CTAS_PER_SM)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    using Cfg = TileConfig<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    __nv_bfloat16* staging = (__nv_bfloat16*)(smem + STAGES * Cfg::STAGE_BYTES + 256);    // [4 warps][32 x 32]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int work_total = p.a_tiles * p.b_tiles * p.splits;

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            // The walk over (work item, block of K) as an iterator, so that the weight tiles of the first stages
            // can be requested before the kernel in front of this one has finished: weights do not depend on it,
            // activations do.
            struct Walk {
                const GemmParams& p;
                int w, kb, kb1, a0, b0;
                bool valid;
                __device__ void start(int w_, int work_total) {
                    w = w_;
                    valid = w < work_total;
                    if (!valid) return;
                    const int split = w % p.splits, tile = w / p.splits;
                    a0 = (tile % p.a_tiles) * BM;
                    b0 = (tile / p.a_tiles) * BN;
                    kb = (int)((long long)p.kblocks * split / p.splits);
                    kb1 = (int)((long long)p.kblocks * (split + 1) / p.splits);
                }
                __device__ void next(int stride, int work_total) { if (++kb == kb1) start(w + stride, work_total); }
            };
            Walk wa{p}, wb{p};
            wa.start(blockIdx.x, work_total);
            wb.start(blockIdx.x, work_total);
            int pre = 0;
            if (p.swapped) {
                // A is the weight: fill the (still empty) ring with weight tiles now
                for (; pre < STAGES && wa.valid; ++pre) {
                    mbar_arrive_expect_tx(&full[pre], Cfg::STAGE_BYTES);
                    tma_load_2d(smem_a + pre * A_BYTES, &map_a, &full[pre], wa.kb * BK, wa.a0);
                    wa.next(gridDim.x, work_total);
                }
            }
            pdl_wait();
            for (int s = 0; s < pre; ++s) {                  // the activation tiles of those stages
                tma_load_2d(smem_b + s * Cfg::B_BYTES, &map_b, &full[s], wb.kb * BK, wb.b0);
                wb.next(gridDim.x, work_total);
            }
            int stage = pre == STAGES ? 0 : pre;
            uint32_t phase = pre == STAGES ? 1 : 0;
            bool ok = true;
            while (wa.valid) {
                if (!mbar_wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_PRODUCER)) { ok = false; break; }
                mbar_arrive_expect_tx(&full[stage], Cfg::STAGE_BYTES);
                tma_load_2d(smem_a + stage * A_BYTES, &map_a, &full[stage], wa.kb * BK, wa.a0);
                tma_load_2d(smem_b + stage * Cfg::B_BYTES, &map_b, &full[stage], wa.kb * BK, wa.b0);
                wa.next(gridDim.x, work_total);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            // Do not leave while copies may still be in flight: wait until the consumer released every stage.
            for (int s = 0; s < STAGES && ok; ++s) {
                if (!mbar_wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_PRODUCER)) break;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < work_total && ok; w += gridDim.x) {
                const int split = w % p.splits;
                const int kb0 = (int)((long long)p.kblocks * split / p.splits);
                const int kb1 = (int)((long long)p.kblocks * (split + 1) / p.splits);
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.error_flag, PH_ERR_WAIT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + (uint32_t)(acc * BN);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, p.error_flag, PH_ERR_WAIT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_smem_desc(smem_u32(smem_a + stage * A_BYTES));
                    const uint64_t bdesc = make_smem_desc(smem_u32(smem_b + stage * Cfg::B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // the next 16 K elements are 32 bytes further along the swizzled row
                        umma_bf16(d_addr, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[stage]);        // frees the stage when these instructions have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);           // the accumulator is complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        const int q = warp & 3;                        // the TMEM lane quarter this warp may read
        pdl_wait();                                    // nothing is written before the kernels in front are done
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < work_total && ok; w += gridDim.x) {
            const int split = w % p.splits, tile = w / p.splits;
            const int a0 = (tile % p.a_tiles) * BM, b0 = (tile / p.a_tiles) * BN;
            constexpr int CH = BN > 64 ? 32 : 16;         // chunks of 16 keep the few-token kernels at registers that let a neighbour start beside them
            // the factors of this item's tokens (register i, lane l: token b0 + 32 i + l), fetched while the products run
            constexpr int FR = BN > 32 ? BN / 32 : 1;
            float factor[FR];
#pragma unroll
            for (int i = 0; i < FR; ++i) {
                factor[i] = 1.0f;
                const int t = b0 + i * 32 + lane;
                if (p.swapped && p.row_sumsq && i * 32 + lane < BN && t < p.rows_b) {
                    float s = 0.0f;
                    for (int k = 0; k < p.row_chunks; ++k) s += p.row_sumsq[(size_t)t * p.row_chunks + k];
                    factor[i] = rsqrtf(s / (float)p.row_width + p.row_eps);
                }
            }
            // plain orientation, tiles of 256 columns: the factor of this thread's row (fetched while the products run), and
            // its sum of squares for the norm ahead
            const int a = a0 + q * 32 + lane;
            constexpr bool ROW_OPS = BN == 256;
            const bool scale_row = ROW_OPS && !p.swapped && p.row_sumsq != nullptr;
            float row_f = 1.0f;
            float ss[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if constexpr (ROW_OPS) row_f = scale_row ? plain_row_factor(p, a) : 1.0f;
            if (!mbar_wait(&acc_full[acc], acc_phase, p.error_flag, PH_ERR_WAIT_EPILOGUE)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            const size_t split_off = (size_t)split * (size_t)p.split_stride;
            // out += product (tiles of 256 columns): the values added to are fetched one chunk ahead
            const bool staged_add = ROW_OPS && !p.swapped && p.accumulate;
            const bool vectors = staged_add && accumulate_in_vectors(p);
            float4 old[ROW_OPS ? 8 : 1], old_next[ROW_OPS ? 8 : 1];
            if constexpr (ROW_OPS) { if (vectors) load_accumulate_chunk(p, a0 + q * 32, lane, b0, 0, old_next); }
#pragma unroll 1
            for (int c = 0; c < BN; c += CH) {
                uint32_t r[CH];
                if constexpr (ROW_OPS) {
                    if (vectors) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) old[i] = old_next[i];
                    }
                }
                if constexpr (CH == 32) tmem_ld32(taddr + c, r); else tmem_ld16(taddr + c, r);
                tmem_ld_wait();
                if constexpr (ROW_OPS) {
                    if (scale_row) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * row_f);
                    }
                }
                if (p.swapped && p.out_bf16) {
                    float f = factor[0];                  // the register that holds this chunk's tokens, picked without an index
#pragma unroll
                    for (int i = 1; i < FR; ++i) if ((c >> 5) == i) f = factor[i];
                    store_chunk_swapped_bf16<CH>(p, r, staging + q * 32 * 32, a0 + q * 32, lane, b0, c, f);
                }
                else if (p.swapped && p.swiglu) store_chunk_swapped_swiglu<CH>(p, r, a, b0, c);
                else if (ROW_OPS && staged_add) {
                    if constexpr (ROW_OPS) {
                        store_chunk_accumulate_staged(p, r, old, vectors, (float*)staging + q * 32 * 32, a0 + q * 32, lane, b0, c, ss,
                                                      old_next, c + CH < BN ? c + CH : -1);
                        if (p.norm_sumsq && ((c + CH) & 127) == 0) store_tile_sumsq(p, ss, a0 + q * 32, lane, 2 * (b0 / BN) + (c >> 7));
                    }
                }
                else store_chunk<CH>(p, r, a, b0, c, split_off);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// ---- two CTAs on one tile (cta_group::2) ---------------------------------------------------------------
//
// Plain orientation, many tokens: a cluster of two CTAs (on the two SMs of a pair) computes one tile of 256
// tokens x 256 features.  Each CTA loads its own 128 rows of A and its own 128 rows of B per block of K (half the
// shared-memory traffic per flop of the one-CTA tile, and six stages instead of four in the same space); the
// leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256, N = 256, which reads A from each
// CTA's own shared memory, B from both, and leaves each CTA's 128 rows x 256 columns of the result in its own
// tensor memory.  Who signals whom:
//   full[s]      in the leader: the copies of both CTAs complete there (TMA .cta_group::2 may complete on the
//                peer's barrier), the leader's producer announces the bytes of both; the leader's MMA thread waits;
//   empty[s]     in each CTA: the leader's tcgen05.commit reaches both (commit's own cluster multicast; no load is
//                multicast);
//   acc_full[a]  in each CTA, by the same kind of commit; acc_empty[a] in the leader, counted in by the eight
//                epilogue warps of both CTAs.
// The cluster is synchronised once after the barriers are initialised and once before tensor memory is freed, so
// that no CTA's shared memory goes away while its peer may still signal it.
constexpr int PAIR_BN = 256;                      // features of the pair's tile
constexpr int PAIR_HALF = PAIR_BN / 2;            // rows of B each CTA loads
constexpr int PAIR_B_BYTES = PAIR_HALF * BK * 2;
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_TMEM_COLS = 2 * PAIR_BN;
constexpr int PAIR_EPILOGUE_WARPS = 8;             // two per quarter of the accumulator's rows, 128 columns each
constexpr int PAIR_THREADS = 64 + 32 * PAIR_EPILOGUE_WARPS;
constexpr int PAIR_STAGING_BYTES = PAIR_EPILOGUE_WARPS * 32 * 32 * 4;        // per epilogue warp: 32 rows x 32 columns, float32
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256 + PAIR_STAGING_BYTES;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of the same location in the CTA of the given rank.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c_inner, int c_row) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c_inner), "r"(c_row) : "memory");
}
// A box from shared memory to its place in the output; the calling thread's bulk group tracks it.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c_inner, int c_row) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c_inner), "r"(c_row) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c_inner, int c_row, int c_outer) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c_inner), "r"(c_row), "r"(c_outer) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Eight bfloat16 values as one 16-byte chunk of row `lane` of a 32 x 64 box laid out as the copy engine's 128-byte
// swizzle wants it (chunk ^ (row & 7)).
__device__ __forceinline__ void put_chunk(unsigned char* box, int lane, int chunk, float v0, float v1, float v2, float v3,
                                          float v4, float v5, float v6, float v7) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v0, v1), b = __floats2bfloat162_rn(v2, v3);
    const __nv_bfloat162 c = __floats2bfloat162_rn(v4, v5), d = __floats2bfloat162_rn(v6, v7);
    *(uint4*)(box + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
        make_uint4(*(const uint32_t*)&a, *(const uint32_t*)&b, *(const uint32_t*)&c, *(const uint32_t*)&d);
}
__device__ __forceinline__ float silu_times(uint32_t g_bits, uint32_t u_bits, float f) {
    const float g = __uint_as_float(g_bits) * f, u = __uint_as_float(u_bits) * f;
    return g / (1.0f + __expf(-g)) * u;
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the MMAs issued so far are complete, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

// ADDS: the instance for out += product (its epilogue keeps two chunks of out in registers); the other instance stores.
template <bool ADDS>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_out, GemmParams p) {
    constexpr int STAGES = PAIR_STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_BYTES;
    float* staging = (float*)(smem + STAGES * PAIR_STAGE_BYTES);             // [epilogue warps][4 KB], 1024-byte aligned
    uint64_t* full = (uint64_t*)(smem + STAGES * PAIR_STAGE_BYTES + PAIR_STAGING_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 2 * PAIR_EPILOGUE_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(PAIR_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int a_tiles = (p.rows_a + 2 * BM - 1) / (2 * BM), b_tiles = (p.rows_b + PAIR_BN - 1) / PAIR_BN;
    const int work_total = a_tiles * b_tiles * p.splits;          // item w: split w % splits of tile w / splits
    const int first = blockIdx.x >> 1, stride = gridDim.x >> 1;
    auto k_range = [&](int w, int& kb0, int& kb1) {
        const int split = w % p.splits;
        kb0 = (int)((long long)p.kblocks * split / p.splits);
        kb1 = (int)((long long)p.kblocks * (split + 1) / p.splits);
    };

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = first; w < work_total && ok; w += stride) {
                const int tile = w / p.splits;
                const int a0 = (tile % a_tiles) * 2 * BM + (int)rank * BM, b0 = (tile / a_tiles) * PAIR_BN + (int)rank * PAIR_HALF;
                int kb0, kb1;
                k_range(w, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_PRODUCER)) { ok = false; break; }
                    const uint32_t bar = cluster_addr(&full[stage], 0);
                    // The leader announces the bytes of both CTAs on its own barrier (a local arrive: one at cluster
                    // scope costs most of a microsecond).  The peer's bytes may land before that: the count of bytes
                    // owed may run negative inside a phase, and the phase still needs the leader's arrival.
                    if (leader) mbar_arrive_expect_tx(&full[stage], 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(smem_a + stage * A_BYTES, &map_a, bar, kb * BK, a0);
                    tma_load_2d_pair(smem_b + stage * PAIR_B_BYTES, &map_b, bar, kb * BK, b0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // Do not leave while copies may still be in flight: wait until the MMAs released every stage.
            for (int s = 0; s < STAGES && ok; ++s) {
                if (!mbar_wait(&empty[stage], phase ^ 1, p.error_flag, PH_ERR_WAIT_PRODUCER)) break;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc(2 * BM, PAIR_BN);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int w = first; w < work_total && ok; w += stride) {
                if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.error_flag, PH_ERR_WAIT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + (uint32_t)(acc * PAIR_BN);
                int kb0, kb1;
                k_range(w, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, p.error_flag, PH_ERR_WAIT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_smem_desc(smem_u32(smem_a + stage * A_BYTES));
                    const uint64_t bdesc = make_smem_desc(smem_u32(smem_b + stage * PAIR_B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(d_addr, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[stage]);       // frees the stage in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[acc]);          // the accumulator halves are complete in both CTAs
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // eight epilogue warps: warp w may read the 32 accumulator rows of quarter w % 4; the two warps of a quarter
        // take 128 columns each, so that the epilogue nothing hides (the last round's) is half as long
        const int q = warp & 3, half = (warp - 2) >> 2, c_first = half * (PAIR_BN / 2);
        pdl_wait();
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int w = first; w < work_total && ok; w += stride) {
            const int tile = w / p.splits;
            const int a0 = (tile % a_tiles) * 2 * BM + (int)rank * BM, b0 = (tile / a_tiles) * PAIR_BN;
            const size_t split_off = (size_t)(w % p.splits) * (size_t)p.split_stride;
            if (!ADDS && p.tma_store) {
                const int a = a0 + q * 32 + lane;
                const float row_f = p.row_sumsq != nullptr ? plain_row_factor(p, a) : 1.0f;   // fetched while the products run
                if (!mbar_wait(&acc_full[acc], acc_phase, p.error_flag, PH_ERR_WAIT_EPILOGUE)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * PAIR_BN);
                // bfloat16 out: the warp's 32 rows x 128 accumulator columns leave as boxes of 64 output columns that
                // the copy engine stores (two boxes, or one with the activation); rows and columns outside of out are
                // clipped by the copy
                unsigned char* box = (unsigned char*)(staging + (warp - 2) * 32 * 32);
                const int row0 = a0 + q * 32;
                if (p.tma_store == 2) {
                    // float32: every chunk of 32 accumulator columns is a box
#pragma unroll 1
                    for (int c = c_first; c < c_first + PAIR_BN / 2; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(taddr + c, r);
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *(float4*)(box + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                                make_float4(__uint_as_float(r[4 * j]) * row_f, __uint_as_float(r[4 * j + 1]) * row_f,
                                            __uint_as_float(r[4 * j + 2]) * row_f, __uint_as_float(r[4 * j + 3]) * row_f);
                        fence_async_shared();
                        __syncwarp();
                        if (lane == 0 && row0 < p.rows_a && b0 + c < p.rows_b) tma_store_3d(&map_out, box, b0 + c, row0, w % p.splits);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[acc], 0));
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                    continue;
                }
                const int boxes = p.swiglu ? 1 : 2, per_box = p.swiglu ? 4 : 2;       // chunks of 32 accumulator columns per box
#pragma unroll 1
                for (int b = 0; b < boxes; ++b) {
                    if (lane == 0) tma_store_wait_read();                          // the box before this one has left shared memory
                    __syncwarp();
#pragma unroll 1
                    for (int k = 0; k < per_box; ++k) {
                        uint32_t r[32];
                        tmem_ld32(taddr + c_first + (b * per_box + k) * 32, r);
                        tmem_ld_wait();
                        if (p.swiglu) {
#pragma unroll
                            for (int j = 0; j < 2; ++j)
                                put_chunk(box, lane, 2 * k + j,
                                          silu_times(r[16 * j], r[16 * j + 1], row_f), silu_times(r[16 * j + 2], r[16 * j + 3], row_f),
                                          silu_times(r[16 * j + 4], r[16 * j + 5], row_f), silu_times(r[16 * j + 6], r[16 * j + 7], row_f),
                                          silu_times(r[16 * j + 8], r[16 * j + 9], row_f), silu_times(r[16 * j + 10], r[16 * j + 11], row_f),
                                          silu_times(r[16 * j + 12], r[16 * j + 13], row_f), silu_times(r[16 * j + 14], r[16 * j + 15], row_f));
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                put_chunk(box, lane, 4 * k + j, __uint_as_float(r[8 * j]) * row_f, __uint_as_float(r[8 * j + 1]) * row_f,
                                          __uint_as_float(r[8 * j + 2]) * row_f, __uint_as_float(r[8 * j + 3]) * row_f,
                                          __uint_as_float(r[8 * j + 4]) * row_f, __uint_as_float(r[8 * j + 5]) * row_f,
                                          __uint_as_float(r[8 * j + 6]) * row_f, __uint_as_float(r[8 * j + 7]) * row_f);
                        }
                    }
                    fence_async_shared();
                    __syncwarp();
                    const int col0 = p.swiglu ? (b0 + c_first) >> 1 : b0 + c_first + b * 64;
                    if (lane == 0 && row0 < p.rows_a && col0 < (int)p.ld) tma_store_2d(&map_out, box, col0, row0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[acc], 0));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                continue;
            }
            // out += product: the values added to are fetched one chunk ahead, the first while the products still run
            const bool vectors = ADDS && accumulate_in_vectors(p);
            float4 old[ADDS ? 8 : 1], old_next[ADDS ? 8 : 1];
            if constexpr (ADDS) { if (vectors) load_accumulate_chunk(p, a0 + q * 32, lane, b0, c_first, old_next); }
            // ... and so is the factor of this thread's row
            const int a = a0 + q * 32 + lane;
            const bool scale_row = !ADDS && p.row_sumsq != nullptr;       // a product that adds takes finished rows
            const float row_f = scale_row ? plain_row_factor(p, a) : 1.0f;
            if (!mbar_wait(&acc_full[acc], acc_phase, p.error_flag, PH_ERR_WAIT_EPILOGUE)) { ok = false; break; }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * PAIR_BN);
            float ss[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
            for (int c = c_first; c < c_first + PAIR_BN / 2; c += 32) {
                uint32_t r[32];
                if constexpr (ADDS) {
                    if (vectors) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) old[i] = old_next[i];
                    }
                }
                tmem_ld32(taddr + c, r);
                tmem_ld_wait();
                if constexpr (!ADDS) {
                    if (scale_row) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * row_f);
                    }
                }
                if constexpr (ADDS) store_chunk_accumulate_staged(p, r, old, vectors, staging + (warp - 2) * 32 * 32, a0 + q * 32, lane, b0, c, ss,
                                                                  old_next, c + 32 < c_first + PAIR_BN / 2 ? c + 32 : -1);
                else store_chunk<32>(p, r, a, b0, c, split_off);
            }
            if constexpr (ADDS) { if (p.norm_sumsq) store_tile_sumsq(p, ss, a0 + q * 32, lane, 2 * (b0 / PAIR_BN) + half); }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_addr(&acc_empty[acc], 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (!ADDS && p.tma_store && lane == 0) tma_store_wait_all();      // the stores of this thread are done before the CTA ends
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                  // nothing of the peer may still reach this CTA
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(PAIR_TMEM_COLS) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------------

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

// A [rows, K] bfloat16 row-major matrix seen as boxes of box_rows x 64 elements, 128-byte swizzle, zero fill
// outside.  Maps are cached: weights and workspace buffers keep their addresses.
bool make_map(CUtensorMap* out, const void* ptr, int rows, int K, int box_rows) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    const auto key = std::make_tuple(ptr, rows, K, box_rows);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
}

// out as float32 [splits][rows][cols] seen as boxes of 32 rows x 32 columns of one split, 128-byte swizzle.
bool make_map_f32_out(CUtensorMap* out, const void* ptr, int rows, int cols, int splits) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    const auto key = std::make_tuple(ptr, rows, cols, splits);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)splits};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)rows * (cuuint64_t)cols * 4};
    const cuuint32_t box[3] = {32, 32, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
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

template <int BN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, int max_ctas, cudaStream_t stream) {
    using Cfg = TileConfig<BN>;
    static bool configured = false;
    auto kernel = gemm_tcgen05_kernel<BN>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return fail(PH_ERR_LAUNCH, "gemm_tcgen05: cannot reserve %d bytes of shared memory", Cfg::SMEM_BYTES);
        configured = true;
    }
    const int work = p.a_tiles * p.b_tiles * p.splits;
    int grid = Cfg::CTAS_PER_SM * sm_count();
    if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
    if (work < grid) grid = work;
    // the staging buffer of the bfloat16 epilogue lies last: launches that do not use it leave it out
    const bool staged = (p.swapped && p.out_bf16) || (!p.swapped && BN == 256 && p.accumulate);
    const size_t bytes = (size_t)Cfg::SMEM_BYTES - (staged ? 0 : Cfg::STAGING_BYTES);
    launch_overlapped(kernel, dim3(grid), dim3(NUM_THREADS), bytes, stream, ma, mb, p);
    return check_launch("gemm_tcgen05");
}

int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& p, int max_clusters,
                cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES) != cudaSuccess)
            return fail(PH_ERR_LAUNCH, "gemm_tcgen05_pair: cannot reserve %d bytes of shared memory", PAIR_SMEM_BYTES);
        configured = true;
    }
    const int work = ((p.rows_a + 2 * BM - 1) / (2 * BM)) * ((p.rows_b + PAIR_BN - 1) / PAIR_BN) * p.splits;
    int clusters = sm_count() / 2;
    if (max_clusters > 0 && max_clusters < clusters) clusters = max_clusters;
    if (work < clusters) clusters = work;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = stream;
    // The cluster kernel is launched in plain stream order, not as a programmatic dependent: started early, under a
    // kernel that still ran, it was seen to stop the device now and then (a step of 512 prompt tokens beside eight
    // decode rows, in two runs of three; never without the early start, never with the one-CTA kernel in its
    // place).  It still lets the kernel behind it start early.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (p.accumulate) { if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<true>, ma, mb, mo, p) != cudaSuccess) {} }
    else if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<false>, ma, mb, mo, p) != cudaSuccess) {}
    return check_launch("gemm_tcgen05_pair");
}

}  // namespace

PH_DEFINE_LAST_ERROR(ph_gemm100)

namespace {
// Plain orientation: why the row operations asked for cannot be done, or null.
const char* row_ops_refused(const float* row_sumsq, int row_chunks, int row_width, const float* norm_weight, const void* norm_rows,
                            const float* norm_sumsq, int splits, int accumulate, int N) {
    if (row_sumsq && (splits > 1 || accumulate || row_chunks < 1 || row_width < 1))
        return "a factor per token goes with one split and without accumulate";
    const int given = (norm_weight != nullptr) + (norm_rows != nullptr) + (norm_sumsq != nullptr);
    if (given == 0) return nullptr;
    if (given != 3) return "norm_weight, norm_rows and norm_sumsq come together";
    if (!accumulate) return "the rows for the norm ahead are written together with the addition into the output";
    if ((N & 3) || (((uintptr_t)norm_weight | (uintptr_t)norm_rows) & 15)) return "the norm ahead needs rows of a multiple of 4 elements and 16-byte aligned arrays";
    return nullptr;
}
}  // namespace

// The same product on pairs of CTAs (tcgen05 cta_group::2): tiles of 256 tokens x 256 features, plain orientation;
// float32 partial results [splits][M, N] with splits > 1.  max_clusters: 0 or a cap on the number of CTA pairs.
// accumulate: out (float32, one split, no activation) += the product.
// row_sumsq .. row_eps: the factor per token that the activations lack (one split, no accumulate); norm_weight [N],
// norm_rows (bfloat16 [M, N]), norm_sumsq (float32 [M, 2 * ceil(N / 256)]): with accumulate, what the norm after this
// addition needs (GemmParams).  All may be null.
PH_EXPORT int ph_gemm_bf16_tcgen05_pair(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K,
                                        int splits, int max_clusters, int swiglu, int accumulate,
                                        const float* row_sumsq, int row_chunks, int row_width, float row_eps,
                                        const float* norm_weight, void* norm_rows, float* norm_sumsq, int* error_flag,
                                        cudaStream_t stream) {
    if (!x || !w || !out || !error_flag || M < 1 || N < 1 || K < 1 || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "gemm_tcgen05_pair: bad arguments (M %d, N %d, K %d)", M, N, K);
    if (K % 8) return fail(PH_ERR_UNSUPPORTED, "gemm_tcgen05_pair: K = %d must be a multiple of 8 (16-byte rows for TMA)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) return fail(PH_ERR_UNSUPPORTED, "gemm_tcgen05_pair: operands must be 16-byte aligned");
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1 || splits > kblocks) return fail(PH_ERR_ARG, "gemm_tcgen05_pair: %d splits for %d blocks of K", splits, kblocks);
    if (splits > 1 && out_dtype != PH_F32) return fail(PH_ERR_ARG, "gemm_tcgen05_pair: partial results are float32");
    if (swiglu && ((N & 1) || splits > 1)) return fail(PH_ERR_ARG, "gemm_tcgen05_pair: the SwiGLU epilogue needs an even N and one split");
    if (accumulate && (swiglu || splits > 1 || out_dtype != PH_F32))
        return fail(PH_ERR_ARG, "gemm_tcgen05_pair: adding into the output needs float32, one split and no activation");
    if (const char* why = row_ops_refused(row_sumsq, row_chunks, row_width, norm_weight, norm_rows, norm_sumsq, splits, accumulate, N))
        return fail(PH_ERR_ARG, "gemm_tcgen05_pair: %s", why);
    CUtensorMap ma, mb;
    if (!make_map(&ma, x, M, K, BM) || !make_map(&mb, w, N, K, PAIR_HALF))
        return fail(PH_ERR_LAUNCH, "gemm_tcgen05_pair: cuTensorMapEncodeTiled failed (rows %d / %d, K %d)", M, N, K);
    GemmParams p;
    p.rows_a = M; p.rows_b = N; p.K = K;
    p.a_tiles = 0; p.b_tiles = (N + PAIR_BN - 1) / PAIR_BN; p.splits = splits; p.kblocks = kblocks;
    p.out = out; p.out_bf16 = out_dtype == PH_BF16; p.swapped = 0; p.swiglu = swiglu; p.accumulate = accumulate; p.ld = swiglu ? N / 2 : N;
    p.split_stride = (long long)M * N; p.error_flag = error_flag;
    p.row_sumsq = row_sumsq; p.row_chunks = row_chunks; p.row_width = row_width; p.row_eps = row_eps;
    p.norm_weight = norm_weight; p.norm_rows = (__nv_bfloat16*)norm_rows; p.norm_sumsq = norm_sumsq;
    // bfloat16 results of whole sums leave through the copy engine where its rules allow (rows of a multiple of 16 bytes)
    CUtensorMap mo = ma;
    p.tma_store = 0;
    if (out_dtype == PH_BF16 && splits == 1 && !accumulate && p.ld % 8 == 0 && (((uintptr_t)out) & 15) == 0 &&
        make_map(&mo, out, M, (int)p.ld, 32))
        p.tma_store = 1;
    else if (out_dtype == PH_F32 && !accumulate && !swiglu && N % 4 == 0 && (((uintptr_t)out) & 15) == 0 &&
             make_map_f32_out(&mo, out, M, N, splits))
        p.tma_store = 2;
    return launch_pair(ma, mb, mo, p, max_clusters, stream);
}

// out[M, N] (or float32 partials [splits][M, N]) = x[M, K] * w[N, K]^T.  swapped: the weight fills the 128-row
// side of the instruction (few tokens); block_n is the tile size on the other side (16 .. 256, a power of two).
// swiglu: the rows of w are (gate, up) pairs and out is [M, N / 2] = silu(gate) * up, computed in the epilogue
// (the formula of src/gpu_ops.hip:103-114 in the reference).
// accumulate: out (float32, plain orientation, one split, no activation) += the product.
// row_sumsq [M][row_chunks] (or null), row_width, row_eps: the activations lack a factor per token, see GemmParams;
// taken by the swapped orientation with bfloat16 output, and by the plain orientation with tiles of 256 columns.
// norm_weight, norm_rows, norm_sumsq: as in the pair kernel (plain orientation, block_n 256, accumulate).
PH_EXPORT int ph_gemm_bf16_tcgen05(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K,
                                   int swapped, int block_n, int splits, int max_ctas, int swiglu, int accumulate,
                                   const float* row_sumsq, int row_chunks, int row_width, float row_eps,
                                   const float* norm_weight, void* norm_rows, float* norm_sumsq,
                                   int* error_flag, cudaStream_t stream) {
    if (!x || !w || !out || !error_flag || M < 1 || N < 1 || K < 1 || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "gemm_tcgen05: bad arguments (M %d, N %d, K %d)", M, N, K);
    if (K % 8) return fail(PH_ERR_UNSUPPORTED, "gemm_tcgen05: K = %d must be a multiple of 8 (16-byte rows for TMA)", K);
    if (((uintptr_t)x | (uintptr_t)w) & 15) return fail(PH_ERR_UNSUPPORTED, "gemm_tcgen05: operands must be 16-byte aligned");
    const int kblocks = (K + BK - 1) / BK;
    if (splits < 1 || splits > kblocks) return fail(PH_ERR_ARG, "gemm_tcgen05: %d splits for %d blocks of K", splits, kblocks);
    if (splits > 1 && out_dtype != PH_F32) return fail(PH_ERR_ARG, "gemm_tcgen05: partial results are float32");
    if (swiglu && (splits > 1 || (N & 1) || (!swapped && block_n < 32)))
        return fail(PH_ERR_ARG, "gemm_tcgen05: the SwiGLU epilogue needs one split, an even N and, in the plain orientation, "
                                "tiles of 32 features or more");
    if (row_sumsq && swapped && (out_dtype != PH_BF16 || splits > 1 || row_chunks < 1 || row_width < 1))
        return fail(PH_ERR_ARG, "gemm_tcgen05: in the swapped orientation a factor per token goes with bfloat16 output and one split");
    if (!swapped) {
        if ((row_sumsq || norm_weight || norm_rows || norm_sumsq) && block_n != 256)
            return fail(PH_ERR_ARG, "gemm_tcgen05: in the plain orientation the row operations go with tiles of 256 columns");
        if (const char* why = row_ops_refused(row_sumsq, row_chunks, row_width, norm_weight, norm_rows, norm_sumsq, splits, accumulate, N))
            return fail(PH_ERR_ARG, "gemm_tcgen05: %s", why);
    } else if (norm_weight || norm_rows || norm_sumsq) {
        return fail(PH_ERR_ARG, "gemm_tcgen05: the rows for the norm ahead are written in the plain orientation only");
    }
    if (accumulate && (swapped || swiglu || splits > 1 || out_dtype != PH_F32))
        return fail(PH_ERR_ARG, "gemm_tcgen05: adding into the output needs the plain orientation, float32, one split and no activation");
    const void* a = swapped ? w : x;
    const void* b = swapped ? x : w;
    const int rows_a = swapped ? N : M, rows_b = swapped ? M : N;
    CUtensorMap ma, mb;
    if (!make_map(&ma, a, rows_a, K, BM) || !make_map(&mb, b, rows_b, K, block_n))
        return fail(PH_ERR_LAUNCH, "gemm_tcgen05: cuTensorMapEncodeTiled failed (rows %d / %d, K %d)", rows_a, rows_b, K);
    GemmParams p;
    p.rows_a = rows_a; p.rows_b = rows_b; p.K = K;
    p.a_tiles = (rows_a + BM - 1) / BM; p.b_tiles = (rows_b + block_n - 1) / block_n;
    p.splits = splits; p.kblocks = kblocks;
    p.out = out; p.out_bf16 = out_dtype == PH_BF16; p.swapped = swapped; p.swiglu = swiglu; p.accumulate = accumulate; p.ld = swiglu ? N / 2 : N;
    p.split_stride = (long long)M * N; p.error_flag = error_flag;
    p.row_sumsq = row_sumsq; p.row_chunks = row_chunks; p.row_width = row_width; p.row_eps = row_eps;
    p.norm_weight = norm_weight; p.norm_rows = (__nv_bfloat16*)norm_rows; p.norm_sumsq = norm_sumsq;
    p.tma_store = 0;
    switch (block_n) {
        case 16: return launch<16>(ma, mb, p, max_ctas, stream);
        case 32: return launch<32>(ma, mb, p, max_ctas, stream);
        case 64: return launch<64>(ma, mb, p, max_ctas, stream);
        case 128: return launch<128>(ma, mb, p, max_ctas, stream);
        case 256: return launch<256>(ma, mb, p, max_ctas, stream);
        default: return fail(PH_ERR_ARG, "gemm_tcgen05: block_n %d is not one of 16, 32, 64, 128, 256", block_n);
    }
}

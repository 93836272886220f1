// Row-wise and element-wise kernels: embedding gather, residual add + RMSNorm, SwiGLU, casts.
//
// The residual stream is float32 in every mode; sums of squares, the residual sum and the activation are
// computed in float32 in a fixed order that depends on the row width only, so a row's result does not
// depend on how many rows the launch has.
//
// Formulas (reference): RMSNorm y = x * rsqrt(mean(x^2) + eps) * w with the add fused in front
// (src/gpu_ops.hip:24-56, 64-101); SwiGLU out = g / (1 + exp(-g)) * u (src/gpu_ops.hip:103-114), here over
// interleaved (gate, up) pairs;
// embedding x[t] = table[token[t]] without scaling (src/qwen_model.cpp:1234-1244).
#include "common.cuh"

namespace {

using namespace ph;

template <typename TT>
__global__ void embed_gather_kernel(const TT* __restrict__ table, const int32_t* __restrict__ ids,
                                    float* __restrict__ out, int E, int V) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);       // ids are validated on the host; never read outside
    const TT* row = table + (size_t)id * E;
    float* o = out + (size_t)t * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = to_float<TT>(row[i]);
}

// One block per output row.  v = x[t] + sum_s add[s][t]; optionally stored back to x; y = rmsnorm(v) * w.
template <typename TA, typename TY, int NT>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ add, int add_splits,
                                   long long add_split_stride, const float* __restrict__ weight, float eps,
                                   const int32_t* __restrict__ rows, int E, TY* __restrict__ y, int write_x) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * E;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < E; i += NT) {
        float v = xr[i];
        if (add) {
            const TA* a = add + (size_t)t * E + i;
            for (int s = 0; s < add_splits; ++s) v += to_float<TA>(a[(size_t)s * add_split_stride]);
            if (write_x) xr[i] = v;
        }
        row_buf[i] = v;
        ss += v * v;
    }
    if (!weight) return;
    const float total = block_sum<NT>(ss, scratch);
    const float inv = rsqrtf(total / (float)E + eps);
    TY* yr = y + (size_t)r * E;
    for (int i = threadIdx.x; i < E; i += NT) yr[i] = from_float<TY>(row_buf[i] * inv * weight[i]);
}

// The same with four consecutive elements per thread and all loads of a row in flight at once: a decode step
// has a handful of rows, so the time of this kernel is the latency of its loads, not their volume.  E % 4 == 0,
// every pointer 16-byte aligned (8 for bfloat16).  The block has ceil(E / 4) threads rounded up to a warp, at
// most 1024; with a thousand rows or more it has 256, so that an SM holds rows in different phases.  The order
// of the additions depends on E only, not on the block's width.
template <typename T> struct Vec4 { };
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

// Partial sums of a split product fetched at once (a decode step's o and down products come in nine parts).  A
// launch with one addend or none takes the kernel made for one: it needs half the registers, and with thousands of
// rows it is the number of resident rows per SM that keeps the memory busy.
constexpr int MANY_PARTS_IN_FLIGHT = 12;

template <typename TA, typename TY, int MAX_IT, int PARTS_IN_FLIGHT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ add, int add_splits,
                                       long long add_split_stride, const float* __restrict__ weight, float eps,
                                       const int32_t* __restrict__ rows, int E, TY* __restrict__ y, int write_x) {
    __shared__ float scratch[128];
    pdl_launch_dependents();
    // what no kernel of this step writes (the norm's weight, the row list) is fetched while the kernel in front
    // still runs
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float4 w[MAX_IT];
#pragma unroll
    for (int it = 0; it < MAX_IT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        w[it] = weight && i < E ? Vec4<float>::load(weight + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    pdl_wait();
    float* xr = x + (size_t)t * E;
    float4 v[MAX_IT];
    float ss[MAX_IT];
#pragma unroll
    for (int it = 0; it < MAX_IT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        ss[it] = 0.0f;
        if (i < E) {
            float4 acc = Vec4<float>::load(xr + i);
            if (add) {
                const TA* a = add + (size_t)t * E + i;
                for (int s0 = 0; s0 < add_splits; s0 += PARTS_IN_FLIGHT) {      // loads in flight, added in order
                    float4 u[PARTS_IN_FLIGHT];
#pragma unroll
                    for (int j = 0; j < PARTS_IN_FLIGHT; ++j)
                        u[j] = s0 + j < add_splits ? Vec4<TA>::load(a + (size_t)(s0 + j) * add_split_stride)
                                                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int j = 0; j < PARTS_IN_FLIGHT; ++j)
                        if (s0 + j < add_splits) { acc.x += u[j].x; acc.y += u[j].y; acc.z += u[j].z; acc.w += u[j].w; }
                }
                if (write_x) Vec4<float>::store(xr + i, acc);
            }
            v[it] = acc;
            ss[it] = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
        }
    }
    if (!weight) return;
    // The sum in an order that the block's width does not change: each run of 32 consecutive vectors by a
    // butterfly, the runs' sums in groups of 32 by another, the groups in turn.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int it = 0; it < MAX_IT; ++it) {
        const float part = warp_sum(ss[it]);
        if (lane == 0) scratch[it * nwarps + warp] = part;
    }
    __syncthreads();
    const int n_parts = (E / 4 + 31) / 32;
    float tot = 0.0f;
    for (int g = 0; g < n_parts; g += 32) tot += warp_sum(g + lane < n_parts ? scratch[g + lane] : 0.0f);
    const float inv = rsqrtf(tot / (float)E + eps);
    TY* yr = y + (size_t)r * E;
#pragma unroll
    for (int it = 0; it < MAX_IT; ++it) {
        const int i = (it * blockDim.x + threadIdx.x) * 4;
        if (i < E)
            Vec4<TY>::store(yr + i, make_float4(v[it].x * inv * w[it].x, v[it].y * inv * w[it].y, v[it].z * inv * w[it].z,
                                                v[it].w * inv * w[it].w));
    }
}

// The same sum with the norm's weight but without the row's factor: v = x + addends (stored back), y = v * weight in the
// output type, and the sum of v^2 over this CTA's chunk of the row in sumsq[row][chunk].  Whoever consumes y applies
// rsqrt(sum over the chunks / E + eps) itself (a product's epilogue, the per-head norm behind the qkv product: the
// factor is one number per row and commutes with the product).  A row is spread over ceil(E / 512) CTAs of 128 threads
// instead of sitting in one, which is what this form is for: few rows, many addends.
constexpr int SUMSQ_CHUNK = 512;

template <typename TA, typename TY>
__global__ void __launch_bounds__(128)
add_weight_sumsq_kernel(float* __restrict__ x, const TA* __restrict__ add, int add_splits, long long add_split_stride,
                        const float* __restrict__ weight, int E, TY* __restrict__ y, float* __restrict__ sumsq) {
    __shared__ float part[4];
    pdl_launch_dependents();
    const int r = blockIdx.x, chunk = blockIdx.y;
    const int i = chunk * SUMSQ_CHUNK + threadIdx.x * 4;
    const float4 w = i < E ? Vec4<float>::load(weight + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    pdl_wait();
    float ss = 0.0f;
    if (i < E) {
        float* xr = x + (size_t)r * E + i;
        float4 acc = Vec4<float>::load(xr);
        if (add) {
            const TA* a = add + (size_t)r * E + i;
            for (int s0 = 0; s0 < add_splits; s0 += MANY_PARTS_IN_FLIGHT) {       // loads in flight, added in order
                float4 u[MANY_PARTS_IN_FLIGHT];
#pragma unroll
                for (int j = 0; j < MANY_PARTS_IN_FLIGHT; ++j)
                    u[j] = s0 + j < add_splits ? Vec4<TA>::load(a + (size_t)(s0 + j) * add_split_stride)
                                               : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int j = 0; j < MANY_PARTS_IN_FLIGHT; ++j)
                    if (s0 + j < add_splits) { acc.x += u[j].x; acc.y += u[j].y; acc.z += u[j].z; acc.w += u[j].w; }
            }
            Vec4<float>::store(xr, acc);
        }
        Vec4<TY>::store(y + (size_t)r * E + i, make_float4(acc.x * w.x, acc.y * w.y, acc.z * w.z, acc.w * w.w));
        ss = acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) sumsq[(size_t)r * gridDim.y + chunk] = ((part[0] + part[1]) + part[2]) + part[3];
}

// SwiGLU over rows laid out [g0, u0, g1, u1, ...] (gate and up rows of the weight interleaved, so that a tile of
// the product holds matching pairs): out[t, j] = silu(g_j) * u_j.  Four outputs per thread when FF % 4 == 0.
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }

template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, int splits, long long split_stride, TO* __restrict__ out,
                              int FF, long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const TI* g = gu + idx * 2;
    float gv = 0.0f, uv = 0.0f;
    for (int s = 0; s < splits; ++s) {
        gv += to_float<TI>(g[(size_t)s * split_stride]);
        uv += to_float<TI>(g[(size_t)s * split_stride + 1]);
    }
    out[idx] = from_float<TO>(silu_mul(gv, uv));
}

template <typename TI, typename TO>
__global__ void swiglu_vec_kernel(const TI* __restrict__ gu, int splits, long long split_stride, TO* __restrict__ out,
                                  long long total4) {
    pdl_launch_dependents();
    pdl_wait();
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;      // group of four outputs
    if (q >= total4) return;
    const TI* src = gu + q * 8;
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b = a;
    for (int s0 = 0; s0 < splits; s0 += 4) {
        float4 u[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const bool on = s0 + j < splits;
            u[2 * j] = on ? Vec4<TI>::load(src + (size_t)(s0 + j) * split_stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            u[2 * j + 1] = on ? Vec4<TI>::load(src + (size_t)(s0 + j) * split_stride + 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (s0 + j < splits) {
                a.x += u[2 * j].x; a.y += u[2 * j].y; a.z += u[2 * j].z; a.w += u[2 * j].w;
                b.x += u[2 * j + 1].x; b.y += u[2 * j + 1].y; b.z += u[2 * j + 1].z; b.w += u[2 * j + 1].w;
            }
    }
    Vec4<TO>::store(out + q * 4, make_float4(silu_mul(a.x, a.y), silu_mul(a.z, a.w), silu_mul(b.x, b.y), silu_mul(b.z, b.w)));
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_float<TO>(to_float<TI>(in[i]));
}

}  // namespace

PH_EXPORT int ph_embed_gather(const void* table, int table_dtype, const int32_t* ids, float* out, int T, int E, int V,
                              cudaStream_t stream) {
    if (!table || !ids || !out || T < 0 || E < 1 || V < 1 || !valid_dtype(table_dtype))
        return fail(PH_ERR_ARG, "embed_gather: bad arguments (T %d, E %d, V %d, dtype %d)", T, E, V, table_dtype);
    if (T == 0) return PH_OK;
    PH_DISPATCH(table_dtype, TT, launch_overlapped(embed_gather_kernel<TT>, dim3(T), dim3(256), 0, stream, (const TT*)table,
                                                   ids, out, E, V));
    return check_launch("embed_gather");
}

PH_EXPORT int ph_add_rmsnorm(float* x, const void* add, int add_dtype, int add_splits, long long add_split_stride,
                             const float* weight, float eps, const int32_t* rows, int n_out, int E, void* y,
                             int y_dtype, int write_x, cudaStream_t stream) {
    if (!x || n_out < 0 || E < 1 || !valid_dtype(add_dtype) || !valid_dtype(y_dtype) || (weight && !y) ||
        (add && add_splits < 1))
        return fail(PH_ERR_ARG, "add_rmsnorm: bad arguments (rows %d, E %d)", n_out, E);
    if (rows && write_x && add) return fail(PH_ERR_ARG, "add_rmsnorm: a gathered launch cannot write x back");
    if (n_out == 0) return PH_OK;
    // vector path: rows of up to 16384 elements, everything 16-byte aligned
    const bool aligned = E % 4 == 0 && E <= 16384 && ((uintptr_t)x & 15) == 0 && (!weight || ((uintptr_t)weight & 15) == 0) &&
                         (!y || ((uintptr_t)y & 15) == 0) && (!add || (((uintptr_t)add & 15) == 0 && add_split_stride % 4 == 0));
    if (aligned) {
        // few rows: as many threads per row as it has vectors (latency); many rows: blocks of 256, so that several
        // rows per SM are in different phases (load, reduce, store) at once
        int threads = ((E / 4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (n_out >= 1024 && E <= 4096 && threads > 256) threads = 256;
        const int iters = (E / 4 + threads - 1) / threads;
#define LAUNCH_VEC(TA, TY, IT)                                                                                          \
        do {                                                                                                            \
            if (!add || add_splits == 1)                                                                                \
                launch_overlapped(add_rmsnorm_vec_kernel<TA, TY, IT, 1>, dim3(n_out), dim3(threads), 0, stream, x,      \
                                  (const TA*)add, add_splits, add_split_stride, weight, eps, rows, E, (TY*)y, write_x); \
            else                                                                                                        \
                launch_overlapped(add_rmsnorm_vec_kernel<TA, TY, IT, MANY_PARTS_IN_FLIGHT>, dim3(n_out), dim3(threads), \
                                  0, stream, x, (const TA*)add, add_splits, add_split_stride, weight, eps, rows, E,     \
                                  (TY*)y, write_x);                                                                     \
        } while (0)
        PH_DISPATCH(add_dtype, TA, PH_DISPATCH(y_dtype, TY, {
            if (iters == 1) LAUNCH_VEC(TA, TY, 1); else if (iters == 2) LAUNCH_VEC(TA, TY, 2); else LAUNCH_VEC(TA, TY, 4);
        }));
#undef LAUNCH_VEC
        return check_launch("add_rmsnorm");
    }
    const size_t smem = (size_t)E * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "add_rmsnorm: width %d exceeds the supported 51200", E);
    constexpr int NT = 256;
#define LAUNCH(TA, TY)                                                                                          \
    do {                                                                                                        \
        auto k = add_rmsnorm_kernel<TA, TY, NT>;                                                                \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        k<<<n_out, NT, smem, stream>>>(x, (const TA*)add, add_splits, add_split_stride, weight, eps, rows, E,   \
                                       (TY*)y, write_x);                                                        \
    } while (0)
    PH_DISPATCH(add_dtype, TA, PH_DISPATCH(y_dtype, TY, LAUNCH(TA, TY)));
#undef LAUNCH
    return check_launch("add_rmsnorm");
}

// x [n_rows, E] float32 += the addends (add_splits partial sums, or none); y = x * weight without the row's factor;
// sumsq [n_rows, chunks] with chunks = ceil(E / 512): the row's sum of squares in parts.  E a multiple of 4 and every
// pointer 16-byte aligned (8 for bfloat16), else refused.
PH_EXPORT int ph_add_weight_sumsq(float* x, const void* add, int add_dtype, int add_splits, long long add_split_stride,
                                  const float* weight, int n_rows, int E, void* y, int y_dtype, float* sumsq, int chunks,
                                  cudaStream_t stream) {
    if (!x || !weight || !y || !sumsq || n_rows < 0 || E < 1 || !valid_dtype(add_dtype) || !valid_dtype(y_dtype) ||
        (add && add_splits < 1))
        return fail(PH_ERR_ARG, "add_weight_sumsq: bad arguments (rows %d, E %d)", n_rows, E);
    if (chunks != (E + SUMSQ_CHUNK - 1) / SUMSQ_CHUNK)
        return fail(PH_ERR_ARG, "add_weight_sumsq: a row of %d elements has %d chunks, not %d", E, (E + SUMSQ_CHUNK - 1) / SUMSQ_CHUNK, chunks);
    if (E % 4 || (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)add) & 15) || (add && add_split_stride % 4))
        return fail(PH_ERR_UNSUPPORTED, "add_weight_sumsq: rows must be a multiple of 4 elements and 16-byte aligned");
    if (n_rows == 0) return PH_OK;
#define LAUNCH_SUMSQ(TA, TY)                                                                                          \
    launch_overlapped(add_weight_sumsq_kernel<TA, TY>, dim3(n_rows, chunks), dim3(128), 0, stream, x, (const TA*)add, \
                      add_splits, add_split_stride, weight, E, (TY*)y, sumsq)
    PH_DISPATCH(add_dtype, TA, PH_DISPATCH(y_dtype, TY, LAUNCH_SUMSQ(TA, TY)));
#undef LAUNCH_SUMSQ
    return check_launch("add_weight_sumsq");
}

PH_EXPORT int ph_swiglu(const void* gate_up, int in_dtype, int splits, long long split_stride, void* out,
                        int out_dtype, int T, int FF, cudaStream_t stream) {
    if (!gate_up || !out || T < 0 || FF < 1 || splits < 1 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "swiglu: bad arguments (T %d, FF %d)", T, FF);
    const long long total = (long long)T * FF;
    if (total == 0) return PH_OK;
    if (FF % 4 == 0 && split_stride % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        const long long total4 = total / 4;
        const unsigned vblocks = (unsigned)((total4 + 255) / 256);
        PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
            launch_overlapped(swiglu_vec_kernel<TI, TO>, dim3(vblocks), dim3(256), 0, stream, (const TI*)gate_up, splits,
                              split_stride, (TO*)out, total4)));
        return check_launch("swiglu");
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
        swiglu_kernel<TI, TO><<<blocks, 256, 0, stream>>>((const TI*)gate_up, splits, split_stride, (TO*)out, FF, total)));
    return check_launch("swiglu");
}

PH_EXPORT int ph_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, cudaStream_t stream) {
    if (!in || !out || n < 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "cast: bad arguments");
    if (n == 0) return PH_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    PH_DISPATCH(in_dtype, TI, PH_DISPATCH(out_dtype, TO,
        cast_kernel<TI, TO><<<blocks, 256, 0, stream>>>((const TI*)in, (TO*)out, n)));
    return check_launch("cast");
}

// y[M, N] = x[M, K] * w[N, K]^T on the CUDA cores, float32 multiply-add, one fixed order.
//
// Every output element is the sum over k = 0, 1, ..., K-1 taken in that order by one thread, whatever M
// and N are and wherever the element lies in its tile, so a row's result does not depend on the batch it
// is in.  No tensor cores and no reduced-precision mode: this is the matrix product of the 32-bit path
// (the reference's exact-order F32 kernels: src/matvec_q.hip:837-991), the plain reference of the
// tensor-core kernels, and the product for shapes they refuse.  x and w may be float32 or bfloat16
// (widened exactly), y float32 or bfloat16.
#include "common.cuh"

namespace {

using namespace ph;

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) gemm_simple_kernel(const TX* __restrict__ x, const TW* __restrict__ w,
                                                          TY* __restrict__ y, int M, int N, int K) {
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / (BN / TN), tc = tid % (BN / TN);      // 16 x 16 threads
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements of each operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx / BK, kk = idx % BK;
            const int k = k0 + kk;
            float xv = 0.0f, wv = 0.0f;
            if (k < K) {
                if (m0 + r < M) xv = to_float<TX>(x[(size_t)(m0 + r) * K + k]);
                if (n0 + r < N) wv = to_float<TW>(w[(size_t)(n0 + r) * K + k]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + tr * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n < N) y[(size_t)m * N + n] = from_float<TY>(acc[i][j]);
        }
    }
}

}  // namespace

PH_EXPORT int ph_gemm_simple(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype, int M,
                             int N, int K, cudaStream_t stream) {
    if (!x || !w || !y || M < 0 || N < 1 || K < 1 || !valid_dtype(x_dtype) || !valid_dtype(w_dtype) ||
        !valid_dtype(y_dtype))
        return fail(PH_ERR_ARG, "gemm_simple: bad arguments (M %d, N %d, K %d)", M, N, K);
    if (M == 0) return PH_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return fail(PH_ERR_UNSUPPORTED, "gemm_simple: %d rows exceed the supported %d", M, 65535 * BM);
#define LAUNCH(TX, TW, TY) \
    gemm_simple_kernel<TX, TW, TY><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, (TY*)y, M, N, K)
    PH_DISPATCH(x_dtype, TX, PH_DISPATCH(w_dtype, TW, PH_DISPATCH(y_dtype, TY, LAUNCH(TX, TW, TY))));
#undef LAUNCH
    return check_launch("gemm_simple");
}

// True 32-bit matrix product  C[M,N] = A[M,K] * W[N,K]^T  on the FP32 pipes (FFMA only: no
// tensor cores, no TF32, no reduced-precision accumulation).  nn.Linear without bias, as
// every projection of the reference is (src/layers/attention.py:62-65, src/layers/swiglu.py:9-11).
//
// Each output element is one chain  acc = fma(a[k], w[k], acc)  for k = 0..K-1 in order.  The
// chain does not depend on M, on the tile the element falls in, or on the other rows, so a
// token's result is bit-equal however the tokens are cut into steps or batches.
//
// A may be float or bfloat16 (converted exactly), C float or bfloat16 (rounded once).

#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 8, THREADS = 256;

template <typename TA, typename TC>
__global__ void __launch_bounds__(THREADS) gemm_f32_kernel(const TA* __restrict__ A, const float* __restrict__ W,
                                                           TC* __restrict__ C, int M, int N, int K, long long lda,
                                                           long long ldw, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int ty = tid / (BN / TN), tx = tid % (BN / TN);
    // loader mapping: 256 threads, each brings 4 consecutive k of one row (BM rows x BK=8 -> 2 threads a row)
    const int lrow = tid >> 1, lk = (tid & 1) * 4;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float av[4], wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lrow, wn = n0 + lrow;
            av[q] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
            wv[q] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            As[lk + q][lrow] = av[q];
            Ws[lk + q][lrow] = wv[q];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(size_t)m * ldc + n] = from_float<TC>(acc[i][j]);
        }
    }
}

}  // namespace

GK_EXPORT int gk_gemm_f32(const void* A, int a_dtype, const float* W, void* C, int c_dtype, int M, int N, int K,
                          long long lda, long long ldw, long long ldc, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(a_dtype) && GK_VALID_DTYPE(c_dtype), "gemm_f32: bad dtype code");
    GK_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    GK_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: a leading dimension is shorter than its row");
    if (M == 0) return GK_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    GK_REQUIRE(grid.y <= 65535u, "gemm_f32: M=%d needs more than 65535 row tiles", M);
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(a_dtype, TA, {
        GK_DISPATCH_DTYPE(c_dtype, TC, {
            gk_launch(gemm_f32_kernel<TA, TC>, grid, dim3(THREADS), 0, s, (const TA*)A, W, (TC*)C, M, N, K, lda, ldw, ldc);
        })
    })
    GK_CHECK_LAUNCH("gemm_f32");
    return GK_OK;
}

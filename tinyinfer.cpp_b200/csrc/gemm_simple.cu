// Plain tiled matrix product on the CUDA cores: C[M,N] (+)= A[M,K] * W[N,K]^T.
//
// This is the true 32-bit path (float32 multiply-add, no tensor cores, no reduced-precision
// mode) and the fallback for operand types or sizes that the tensor-core kernels refuse.
// Operands may be float32 or bfloat16 in any combination (widening bfloat16 is exact); the
// product is accumulated in float32 with one fused multiply-add per term, k ascending, so an
// output element's value does not depend on M, on the tile it falls in or on its neighbours.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename TA, typename TW>
__global__ void __launch_bounds__(THREADS)
gemm_tiled_kernel(const TA* __restrict__ a, const TW* __restrict__ w, float* __restrict__ c,
                  int m, int n, int k, int lda, int ldw, int ldc, int accumulate) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kk = k0 + lk + j;
            const int am = m0 + lrow, wn = n0 + lrow;
            as[lk + j][lrow] = (am < m && kk < k) ? to_f32(a[(size_t)am * lda + kk]) : 0.0f;
            ws[lk + j][lrow] = (wn < n && kk < k) ? to_f32(w[(size_t)wn * ldw + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = m0 + ty * 4 + i;
        if (row >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + tx * 4 + j;
            if (col >= n) continue;
            float* p = c + (size_t)row * ldc + col;
            *p = accumulate ? *p + acc[i][j] : acc[i][j];
        }
    }
}

template <typename TA, typename TW>
int launch(const void* a, const void* w, float* c, int m, int n, int k, int lda, int ldw, int ldc,
           int accumulate, cudaStream_t s) {
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    gemm_tiled_kernel<TA, TW><<<grid, THREADS, 0, s>>>((const TA*)a, (const TW*)w, c, m, n, k, lda,
                                                       ldw, ldc, accumulate);
    return ti_check_launch("gemm_simple");
}

}  // namespace

extern "C" int ti_gemm_simple(const void* a, int a_dtype, const void* w, int w_dtype, float* c,
                              int m, int n, int k, int lda, int ldw, int ldc, int accumulate,
                              void* stream) {
    if (m == 0 || n == 0) return 0;
    TI_REQUIRE(k > 0, "gemm: inner size %d", k);
    TI_REQUIRE((m + BM - 1) / BM <= 65535, "gemm: %d rows exceed the grid limit", m);
    cudaStream_t s = (cudaStream_t)stream;
    if (a_dtype == TI_F32 && w_dtype == TI_F32)
        return launch<float, float>(a, w, c, m, n, k, lda, ldw, ldc, accumulate, s);
    if (a_dtype == TI_F32 && w_dtype == TI_BF16)
        return launch<float, bf16>(a, w, c, m, n, k, lda, ldw, ldc, accumulate, s);
    if (a_dtype == TI_BF16 && w_dtype == TI_F32)
        return launch<bf16, float>(a, w, c, m, n, k, lda, ldw, ldc, accumulate, s);
    if (a_dtype == TI_BF16 && w_dtype == TI_BF16)
        return launch<bf16, bf16>(a, w, c, m, n, k, lda, ldw, ldc, accumulate, s);
    return ti_fail("gemm: dtype codes %d x %d are not float32/bfloat16", a_dtype, w_dtype);
}

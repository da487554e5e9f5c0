// C[M,N] = A[M,K] * W[N,K]^T (+ bias), true 32-bit: float inputs (weights may be stored as
// bfloat16 and are widened exactly), FFMA accumulation, no tensor-core mode of reduced precision.
//
// Every output element is one chain of fmaf over k = 0..K-1 in ascending order, whatever M is
// and wherever the element falls in a tile; a row's result therefore does not depend on which
// other rows share the launch.  This is the matrix product of the 32-bit engine; the bfloat16
// engine's products use tensor cores.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TW>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const TW* __restrict__ W, int ldw,
                const TW* __restrict__ bias, float* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per tile, 256 threads: 4 each; consecutive threads walk k (contiguous)
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = threadIdx.x + it * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f<TW>(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j] + (bias ? to_f<TW>(bias[gn]) : 0.f);
        }
    }
}

TL_EXPORT int tl_gemm_f32(const float* A, int lda, const void* W, int ldw, int w_dtype, const void* bias,
                          float* C, int ldc, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return 1;
    if (w_dtype == TL_F32)
        gemm_f32_kernel<float><<<grid, 256, 0, stream>>>(A, lda, (const float*)W, ldw, (const float*)bias, C, ldc, M, N, K);
    else
        gemm_f32_kernel<bf16><<<grid, 256, 0, stream>>>(A, lda, (const bf16*)W, ldw, (const bf16*)bias, C, ldc, M, N, K);
    return tl_launch_status();
}

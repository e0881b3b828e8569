// C[M,N] = alpha * A[M,K] * W[N,K]^T in true fp32: fp32 operands, fp32 FMA, no
// tensor cores and no reduced-precision matrix mode.  It is the matrix product of
// the 32-bit path (the reference has only 16-bit instantiations and cuBLAS,
// src/model/linear.cuh:8-37).  The sum over K runs in the same order for every row,
// whatever M is, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc, float alpha) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;            // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // each thread loads 4 elements of A and 4 of W: element e = tid + 256*i -> (row e/16, k e%16)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + 256 * i;
            const int r = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            const int am = m0 + r, wn = n0 + r;
            As[kk][r] = (am < M && k < K) ? A[(int64_t)am * lda + k] : 0.f;
            Ws[kk][r] = (wn < N && k < K) ? W[(int64_t)wn * ldw + k] : 0.f;
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
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)m * ldc + n] = alpha * acc[i][j];
        }
    }
}

CPM_API int cpm_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int64_t lda,
                         int64_t ldw, int64_t ldc, float alpha, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return CPM_OK;
    if (K <= 0) return CPM_BAD_ARGUMENT;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc, alpha);
    return launch_status();
}

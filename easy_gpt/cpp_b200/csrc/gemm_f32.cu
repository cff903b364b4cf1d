// True float32 matrix product for the 32-bit path:  C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]).
// Plain FFMA on the CUDA cores: no tensor cores, no TF32, no split-K.  Each
// output element is one thread's sum over k in ascending order, so its value
// does not depend on M, i.e. on how tokens were batched.  (The reference's
// Linear is the same contraction with float32 accumulation, src/ops.cpp:79-121.)
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
}

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                   const float* __restrict__ bias, float* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements per operand tile, 256 threads: 4 elements each
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int row = e / BK, col = e % BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + col;
            As[col][row] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.0f;
            Ws[col][row] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            C[(size_t)gm * ldc + gn] = v;
        }
    }
}

EG_API int eg_gemm_f32_nt(cudaStream_t stream, const float* A, int lda, const float* W, int ldw, const float* bias,
                          float* C, int ldc, int M, int N, int K) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, bias, C, ldc, M, N, K);
    return eg_launch_status();
}

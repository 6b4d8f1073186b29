// True 32-bit matrix product for the float32 path: C[M,N] = A[M,K] . W[N,K]^T
// with W stored [out, in] as in the checkpoint (gemvNT, model/llama.go:1516-1536).
// CUDA cores only, fmaf accumulation, no TF32 and no reduced-precision mode.
// Every output element is one accumulator that walks k = 0..K-1 in order, so
// its value does not depend on M, on the tile it falls in, or on what else is
// in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, const float* __restrict__ W, int ldw,
                float* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid >> 2, lk = (tid & 3) * 4;   // loader: 64 rows x 4 chunks of 4 k
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + j][lrow] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
            Ws[lk + j][lrow] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
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
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}
}  // namespace

GTG_API int gtg_gemm_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                         int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return kErrBadArgument;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return kErrUnsupported;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, lda, W, ldw, C, ldc, M, N, K);
    return launch_status();
}

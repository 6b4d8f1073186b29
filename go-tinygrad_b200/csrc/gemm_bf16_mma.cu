// General bfloat16 matrix product on the warp-level tensor-core path:
//   C[M,N] = A[M,K] . W[N,K]^T,  float accumulation, output bfloat16 or float.
// W is stored [out, in] as in the checkpoint.  Any M and N; K a multiple of 8
// (16-byte rows).  This is the route for shapes the tcgen05 kernel refuses and
// the comparison point for it; 128x128x32 tiles, four cp.async stages,
// ldmatrix + mma.sync.m16n8k16.
#include "mma_helpers.cuh"

namespace {
constexpr int BM = 128, BN = 128, BK = 32, STAGES = 4;
constexpr int kThreads = 256;
constexpr int kStageBytes = (BM + BN) * BK * 2;

template <typename OutT>
__device__ __forceinline__ void store_pair(OutT* C, int ldc, int m, int n, int M, int N, float v0, float v1, bool vec_ok);

template <>
__device__ __forceinline__ void store_pair<bf16>(bf16* C, int ldc, int m, int n, int M, int N, float v0, float v1, bool vec_ok) {
    if (m >= M || n >= N) return;
    bf16* p = C + (size_t)m * ldc + n;
    if (vec_ok && n + 1 < N) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v0, v1);
    } else {
        p[0] = __float2bfloat16_rn(v0);
        if (n + 1 < N) p[1] = __float2bfloat16_rn(v1);
    }
}

template <>
__device__ __forceinline__ void store_pair<float>(float* C, int ldc, int m, int n, int M, int N, float v0, float v1, bool vec_ok) {
    if (m >= M || n >= N) return;
    float* p = C + (size_t)m * ldc + n;
    if (vec_ok && n + 1 < N) {
        *reinterpret_cast<float2*>(p) = make_float2(v0, v1);
    } else {
        p[0] = v0;
        if (n + 1 < N) p[1] = v1;
    }
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads)
gemm_bf16_mma_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, int ldw,
                     OutT* __restrict__ C, int ldc, int M, int N, int K) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;          // 2 x 4 warps, 64 x 32 each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const uint32_t smem_base = smem_u32(smem);
    const int nk = (K + BK - 1) / BK;

    auto load_stage = [&](int stage, int kt) {
        const uint32_t a_base = smem_base + stage * kStageBytes;
        const uint32_t w_base = a_base + BM * BK * 2;
        const int k0 = kt * BK;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int id = tid + i * kThreads;       // 512 chunks per operand
            const int r = id >> 2, c = id & 3;
            const int k = k0 + c * 8;
            {
                const int m = m0 + r;
                const bool ok = m < M && k < K;
                const bf16* src = ok ? A + (size_t)m * lda + k : A;
                cp_async16(a_base + swz_offset<BK>(r, c), src, ok ? 16 : 0);
            }
            {
                const int n = n0 + r;
                const bool ok = n < N && k < K;
                const bf16* src = ok ? W + (size_t)n * ldw + k : W;
                cp_async16(w_base + swz_offset<BK>(r, c), src, ok ? 16 : 0);
            }
        }
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < nk) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < nk; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nxt = kt + STAGES - 1;
            if (nxt < nk) load_stage(nxt % STAGES, nxt);
            cp_async_commit();
        }
        const uint32_t a_base = smem_base + (kt % STAGES) * kStageBytes;
        const uint32_t w_base = a_base + BM * BK * 2;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t af[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = wm * 64 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], a_base + swz_offset<BK>(r, c));
            }
            uint32_t bfr[4][2];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int r = wn * 32 + jj * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bfr[jj * 2][0], bfr[jj * 2][1], bfr[jj * 2 + 1][0], bfr[jj * 2 + 1][1],
                            w_base + swz_offset<BK>(r, c));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], af[i], bfr[j][0], bfr[j][1]);
        }
    }
    cp_async_wait<0>();

    const int g = lane >> 2, t = lane & 3;
    const bool vec_ok = (ldc % 2 == 0) && ((reinterpret_cast<uintptr_t>(C) % (2 * sizeof(OutT))) == 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + wm * 64 + i * 16 + g;
            const int n = n0 + wn * 32 + j * 8 + t * 2;
            store_pair<OutT>(C, ldc, m, n, M, N, acc[i][j][0], acc[i][j][1], vec_ok);
            store_pair<OutT>(C, ldc, m + 8, n, M, N, acc[i][j][2], acc[i][j][3], vec_ok);
        }
    }
}
}  // namespace

GTG_API int gtg_gemm_bf16_mma(const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                              int out_f32, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return kErrBadArgument;
    if (K % 8 || lda % 8 || ldw % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return kErrUnsupported;
    const int smem = STAGES * kStageBytes;
    cudaError_t e;
    static bool configured = false;
    if (!configured) {
        e = cudaFuncSetAttribute(gemm_bf16_mma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gemm_bf16_mma_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (out_f32) {
        gemm_bf16_mma_kernel<float><<<grid, kThreads, smem, stream>>>((const bf16*)A, lda, (const bf16*)W, ldw, (float*)C, ldc, M, N, K);
    } else {
        gemm_bf16_mma_kernel<bf16><<<grid, kThreads, smem, stream>>>((const bf16*)A, lda, (const bf16*)W, ldw, (bf16*)C, ldc, M, N, K);
    }
    return launch_status();
}

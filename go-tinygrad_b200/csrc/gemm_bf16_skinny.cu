// Weight-streaming bfloat16 product for decode steps: C[M,N] = X[M,K] . W[N,K]^T
// with few rows M (one token per live sequence, M <= 64).  The work is reading W
// once from HBM; everything is shaped around that.
//
//   * One CTA owns 16 output features (rows of W): they are the M dimension of
//     mma.sync.m16n8k16, the tokens are its N dimension (8 per tile).
//   * The CTA's 8 warps split K: warp w takes the 32-wide k blocks w, w+8, ...,
//     so at any moment the CTA reads one contiguous 512-byte stretch of each
//     row.  Each thread loads 16 bytes (8 consecutive k) of rows g and g+8; the
//     MMA's k slots are assigned to those 8 values in the order they lie in
//     memory (a dot product does not care about the order of k as long as both
//     operands agree), so no shuffle or shared-memory staging is needed.
//   * Four k blocks are in flight per thread (8 x 16-byte loads of W), W bypasses
//     L1 (read once), X stays in L1/L2 (read by every CTA).
//   * The 8 partial sums of an output are added in warp order through shared
//     memory: the result does not depend on timing.
// Any N; K a multiple of 8; output bfloat16 or float.
#include "mma_helpers.cuh"

namespace {
constexpr int kWarps = 8;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

template <int NT, typename OutT>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(const bf16* __restrict__ X, int ldx, const bf16* __restrict__ W, int ldw,
                   OutT* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float red[kWarps][16][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);     // clamped: extra rows are dropped at the store
    const bf16* w0 = W + (size_t)r0 * ldw + t * 8;
    const bf16* w1 = W + (size_t)r1 * ldw + t * 8;
    const bf16* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xrow[j] = X + (size_t)min(j * 8 + g, M - 1) * ldx + t * 8;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

    const int nkb = (K + 31) / 32;
    for (int kb = warp; kb < nkb; kb += kWarps * kUnroll) {
        uint4 wa[kUnroll], wb[kUnroll];
        bool ok[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (kb + u * kWarps) * 32;
            ok[u] = (kb + u * kWarps) < nkb && (k + t * 8) < K;
            wa[u] = ok[u] ? ld_stream16(w0 + k) : make_uint4(0, 0, 0, 0);
            wb[u] = ok[u] ? ld_stream16(w1 + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int k = (kb + u * kWarps) * 32;
            const uint32_t a_lo[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y};
            const uint32_t a_hi[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 xb = ok[u] ? ld_cached16(xrow[j] + k) : make_uint4(0, 0, 0, 0);
                mma_bf16_16816(acc[j], a_lo, xb.x, xb.y);
                mma_bf16_16816(acc[j], a_hi, xb.z, xb.w);
            }
        }
    }
    // acc[j][0,1]: feature g, tokens 8j+2t, +1;  acc[j][2,3]: feature g+8, same tokens
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][g][j * 8 + t * 2] = acc[j][0];
        red[warp][g][j * 8 + t * 2 + 1] = acc[j][1];
        red[warp][g + 8][j * 8 + t * 2] = acc[j][2];
        red[warp][g + 8][j * 8 + t * 2 + 1] = acc[j][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kWarps * 32) {
        const int m = idx >> 4, r = idx & 15;          // consecutive threads -> consecutive features
        if (m >= M || n0 + r >= N) continue;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[w][r][m];
        C[(size_t)m * ldc + n0 + r] = from_f32<OutT>(s);
    }
}

template <int NT>
int launch(const bf16* X, int ldx, const bf16* W, int ldw, void* C, int ldc, int out_f32,
           int M, int N, int K, cudaStream_t stream) {
    const int blocks = (N + 15) / 16;
    if (out_f32)
        gemm_skinny_kernel<NT, float><<<blocks, kWarps * 32, 0, stream>>>(X, ldx, W, ldw, (float*)C, ldc, M, N, K);
    else
        gemm_skinny_kernel<NT, bf16><<<blocks, kWarps * 32, 0, stream>>>(X, ldx, W, ldw, (bf16*)C, ldc, M, N, K);
    return launch_status();
}
}  // namespace

// Rows (tokens) this kernel takes.
GTG_API int gtg_gemm_bf16_skinny_max_rows() { return 64; }

GTG_API int gtg_gemm_bf16_skinny(const void* X, int ldx, const void* W, int ldw, void* C, int ldc,
                                 int out_f32, int M, int N, int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || ldx < K || ldw < K || ldc < N) return kErrBadArgument;
    if (M > 64) return kErrUnsupported;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (M <= 8) return launch<1>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, stream);
    if (M <= 16) return launch<2>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, stream);
    if (M <= 32) return launch<4>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, stream);
    return launch<8>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, stream);
}

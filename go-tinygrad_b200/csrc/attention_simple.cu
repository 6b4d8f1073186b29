// Causal grouped-query attention over the paged cache, one warp per
// (token, query head).  This is the attention of the float32 path (and the
// bfloat16 path's route for head sizes its tiled kernels refuse).  It serves a
// prompt and a decode step alike: token n at position p sees keys lo..p of its
// own sequence, lo = 0 or p-window+1.
//
// Scores are (q.k)*scale with the scale applied after the dot; softmax is the
// streaming form of max / exp / sum / normalise (model/llama.go:1626-1660), with
// expf, never a fast approximation.  Keys are walked 32 at a time from lo, so
// the value for a (token, head) depends on nothing but its own keys: not on the
// batch, not on how the tokens were cut into steps.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int kWarps = 4;
constexpr int kMaxPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attention_simple_kernel(const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo,
                        const T* __restrict__ kc, const T* __restrict__ vc, long long page_stride,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ token_seq, const int* __restrict__ slots,
                        const int* __restrict__ positions,
                        int N, int n_heads, int n_kv, int hd, float scale, int window) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * kWarps + warp;
    if (wid >= (long long)N * n_heads) return;
    const int n = (int)(wid / n_heads), h = (int)(wid % n_heads);
    const int kvh = h / (n_heads / n_kv);
    const int pos = positions[n];
    const int slot = slots[token_seq[n]];
    const int* table = block_table + (size_t)slot * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float* qs = smem + warp * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = to_f32<T>(q[(size_t)n * ldq + h * hd + d]);
    __syncwarp();

    float acc[kMaxPerLane];
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int t0 = lo; t0 <= pos; t0 += 32) {
        const int t = t0 + lane;
        const bool valid = t <= pos;
        int page = 0;
        float score = -INFINITY;
        if (valid) {
            page = table[t / kPageTokens];
            const T* kp = kc + (size_t)page * page_stride + ((size_t)kvh * kPageTokens + (t % kPageTokens)) * hd;
            float s = 0.f;
            for (int d = 0; d < hd; ++d) s = fmaf(qs[d], to_f32<T>(kp[d]), s);
            score = s * scale;
        }
        const float m_new = fmaxf(m, warp_max(score));
        const float p = valid ? expf(score - m_new) : 0.f;
        const float corr = expf(m - m_new);      // 0 on the first chunk (m = -inf)
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) acc[j] *= corr;
        const int count = min(32, pos - t0 + 1);
        for (int src = 0; src < count; ++src) {
            const float pj = __shfl_sync(0xffffffffu, p, src);
            const int pg = __shfl_sync(0xffffffffu, page, src);
            const int tj = t0 + src;
            const T* vp = vc + (size_t)pg * page_stride + ((size_t)kvh * kPageTokens + (tj % kPageTokens)) * hd;
#pragma unroll
            for (int j = 0; j < kMaxPerLane; ++j) {
                const int d = lane + 32 * j;
                if (d < hd) acc[j] = fmaf(pj, to_f32<T>(vp[d]), acc[j]);
            }
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) out[(size_t)n * ldo + h * hd + d] = from_f32<T>(acc[j] * inv);
    }
}
}  // namespace

GTG_API int gtg_attention_simple(int dtype, const void* q, int ldq, void* out, int ldo,
                                 const void* kc, const void* vc, long long page_stride,
                                 const int* block_table, int table_stride,
                                 const int* token_seq, const int* slots, const int* positions,
                                 int N, int n_heads, int n_kv, int hd, float scale, int window,
                                 cudaStream_t stream) {
    if (N <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || hd <= 0) return kErrBadArgument;
    if (hd > 32 * kMaxPerLane) return kErrUnsupported;
    const long long warps = (long long)N * n_heads;
    const long long blocks = (warps + kWarps - 1) / kWarps;
    if (blocks > 0x7fffffffLL) return kErrUnsupported;
    const size_t smem = (size_t)kWarps * hd * sizeof(float);
    if (dtype == 0)
        attention_simple_kernel<float><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(
            (const float*)q, ldq, (float*)out, ldo, (const float*)kc, (const float*)vc, page_stride,
            block_table, table_stride, token_seq, slots, positions, N, n_heads, n_kv, hd, scale, window);
    else if (dtype == 1)
        attention_simple_kernel<bf16><<<(unsigned)blocks, kWarps * 32, smem, stream>>>(
            (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kc, (const bf16*)vc, page_stride,
            block_table, table_stride, token_seq, slots, positions, N, n_heads, n_kv, hd, scale, window);
    else return kErrBadArgument;
    return launch_status();
}

// Token selection from float32 logits, one block per row.
//   greedy:      the first index of the maximum (strict '>' scan, lowest index
//                wins ties: model/inference_helpers.go:153-166)
//   temperature: p = softmax(logits / T) with float statistics, then the first
//                token whose cumulative probability exceeds u, where u is a
//                counter-based uniform that depends on (seed, sequence id,
//                step) only -- never on what else is in the batch.
// The reference samples greedily only; temperature sampling is this library's.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int kThreads = 256;

constexpr int kArgmaxThreads = 1024;

// (a, ia) <- the better of (a, ia) and (b, ib): the larger value, the lower index on a tie.
__device__ __forceinline__ void argmax_merge(float& a, int& ia, float b, int ib) {
    if (b > a || (b == a && ib < ia)) { a = b; ia = ib; }
}

// One block per row; each thread scans its elements in increasing index order
// (16 bytes at a time when the row allows it), then warps and the block merge.
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
    chain_release();
    chain_wait();
    __shared__ float bv[kArgmaxThreads / 32];
    __shared__ int bi[kArgmaxThreads / 32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = V;                      // "nothing yet": any real index beats it on a tie
    auto see = [&](float v, int i) {
        if (v > best || (idx == V && !(v != v))) { best = v; idx = i; }
    };
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int V4 = vec ? V / 4 : 0;
    for (int i = threadIdx.x; i < V4; i += kArgmaxThreads) {
        const float4 v = reinterpret_cast<const float4*>(row)[i];
        see(v.x, 4 * i); see(v.y, 4 * i + 1); see(v.z, 4 * i + 2); see(v.w, 4 * i + 3);
    }
    for (int i = 4 * V4 + threadIdx.x; i < V; i += kArgmaxThreads) see(row[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_merge(best, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = bv[threadIdx.x];
        idx = bi[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_merge(best, idx, ov, oi);
        }
        if (threadIdx.x == 0) out[blockIdx.x] = idx < V ? idx : 0;
    }
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// 24 random bits as a float in [0, 1).
__device__ __forceinline__ float uniform24(unsigned long long seed, int sequence, int step) {
    unsigned long long z = mix64(seed);
    z = mix64(z ^ ((unsigned long long)(long long)sequence * 0xD1B54A32D192ED03ull));
    z = mix64(z ^ ((unsigned long long)(long long)step * 0x8CB92BA72F3D8DD7ull));
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kThreads)
sample_temperature_kernel(const float* __restrict__ logits, int ld, int V, float inv_temperature,
                          unsigned long long seed, const int* __restrict__ sequence_ids,
                          const int* __restrict__ steps, int* __restrict__ out) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    __shared__ float seg_sum[kThreads];
    __shared__ int chosen_seg;
    __shared__ float chosen_prefix;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int tid = threadIdx.x;

    float mx = -INFINITY;
    for (int i = tid; i < V; i += kThreads) mx = fmaxf(mx, row[i] * inv_temperature);
    mx = warp_max(mx);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = mx;
    __syncthreads();
    mx = scratch[0];
    for (int w = 1; w < kThreads / 32; ++w) mx = fmaxf(mx, scratch[w]);
    __syncthreads();

    // Each thread owns one contiguous segment of the vocabulary, so that the
    // cumulative sum below runs in vocabulary order.
    const int seg = (V + kThreads - 1) / kThreads;
    const int begin = min(V, tid * seg), end = min(V, begin + seg);
    float s = 0.f;
    for (int i = begin; i < end; ++i) s += expf(row[i] * inv_temperature - mx);
    seg_sum[tid] = s;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int t = 0; t < kThreads; ++t) total += seg_sum[t];
        const float target = uniform24(seed, sequence_ids[r], steps[r]) * total;
        float prefix = 0.f;
        int pick = -1, last_nonempty = 0;
        float last_prefix = 0.f;
        for (int t = 0; t < kThreads; ++t) {
            if (seg_sum[t] > 0.f) { last_nonempty = t; last_prefix = prefix; }
            if (target < prefix + seg_sum[t]) { pick = t; break; }
            prefix += seg_sum[t];
        }
        if (pick < 0) { pick = last_nonempty; prefix = last_prefix; }
        chosen_seg = pick;
        chosen_prefix = prefix;
        scratch[32] = target;
    }
    __syncthreads();
    if (tid == chosen_seg) {
        const float target = scratch[32];
        float c = chosen_prefix;
        int pick = -1, last_positive = begin;
        for (int i = begin; i < end; ++i) {
            const float e = expf(row[i] * inv_temperature - mx);
            if (e > 0.f) last_positive = i;
            c += e;
            if (c > target) { pick = i; break; }
        }
        out[r] = pick >= 0 ? pick : last_positive;
    }
}
}  // namespace

GTG_API int gtg_argmax(const float* logits, int ld, int R, int V, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return kErrBadArgument;
    return launch_chained(argmax_kernel, dim3(R), dim3(kArgmaxThreads), 0, stream, logits, ld, V, out);
}

GTG_API int gtg_sample_temperature(const float* logits, int ld, int R, int V, float temperature,
                                   unsigned long long seed, const int* sequence_ids,
                                   const int* steps, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || !(temperature > 0.f)) return kErrBadArgument;
    return launch_chained(sample_temperature_kernel, dim3(R), dim3(kThreads), 0, stream, logits, ld, V,
                          1.0f / temperature, seed, sequence_ids, steps, out);
}

// Token selection from float32 logits: one block per row, or for long rows a
// cluster of up to eight blocks that share the row and meet through the
// cluster's shared memory (one block reads a row at a few tens of GB/s; a
// vocabulary of 128k entries would take it 20 us to scan once).
//   greedy:      the first index of the maximum (strict '>' scan, lowest index
//                wins ties: model/inference_helpers.go:153-166)
//   temperature: p = softmax(logits / T) with float statistics, then the first
//                token whose cumulative probability exceeds u, where u is a
//                counter-based uniform that depends on (seed, sequence id,
//                step) only -- never on what else is in the batch.
// The reference samples greedily only; temperature sampling is this library's.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>

namespace cg = cooperative_groups;

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

// ------------------------------------------------------------ rows over a cluster
constexpr int kRowThreads = 512;
constexpr int kMaxRanks = 8;
constexpr int kChunkFloats = 16384;          // of a row per block: what the sampler keeps in shared memory

// Blocks of the cluster that share a row of V entries (a power of two up to 8), and
// each block's share of it, a multiple of 4 entries.
static int row_ranks(int V, int per_block) {
    int c = 1;
    while (c < kMaxRanks && (V + c - 1) / c > per_block) c *= 2;
    return c;
}
__device__ __forceinline__ int row_chunk(int V, int ranks) { return ((V + ranks - 1) / ranks + 3) / 4 * 4; }

// grid (ranks, rows), clusters of `ranks` blocks along x.  Each block scans its
// chunk of the row (every thread in increasing index order, four 16-byte loads in
// flight), the blocks' candidates meet in the first block, which takes the largest
// value and on a tie the lowest index.
__global__ void __launch_bounds__(kRowThreads)
argmax_cluster_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
    chain_release();
    chain_wait();
    __shared__ float bv[kRowThreads / 32];
    __shared__ int bi[kRowThreads / 32];
    __shared__ float cand_v[kMaxRanks];
    __shared__ int cand_i[kMaxRanks];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), ranks = (int)cluster.num_blocks();
    const float* row = logits + (size_t)blockIdx.y * ld;
    const int chunk = row_chunk(V, ranks);
    const int begin = min(V, rank * chunk), end = min(V, begin + chunk);
    float best = -INFINITY;
    int idx = V;                      // "nothing yet": any real index beats it on a tie
    auto see = [&](float v, int i) {
        if (v > best || (idx == V && !(v != v))) { best = v; idx = i; }
    };
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int q_begin = begin / 4, q_end = vec ? end / 4 : q_begin;      // whole groups of four
    int i = q_begin + threadIdx.x;
    for (; i + 3 * kRowThreads < q_end; i += 4 * kRowThreads) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = reinterpret_cast<const float4*>(row)[i + u * kRowThreads];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int at = 4 * (i + u * kRowThreads);
            see(v[u].x, at); see(v[u].y, at + 1); see(v[u].z, at + 2); see(v[u].w, at + 3);
        }
    }
    for (; i < q_end; i += kRowThreads) {
        const float4 v = reinterpret_cast<const float4*>(row)[i];
        see(v.x, 4 * i); see(v.y, 4 * i + 1); see(v.z, 4 * i + 2); see(v.w, 4 * i + 3);
    }
    for (int k = (vec ? 4 * q_end : begin) + threadIdx.x; k < end; k += kRowThreads) see(row[k], k);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_merge(best, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < kRowThreads / 32 ? bv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < kRowThreads / 32 ? bi[threadIdx.x] : V;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            argmax_merge(best, idx, ov, oi);
        }
        if (threadIdx.x == 0) {
            *cluster.map_shared_rank(&cand_v[rank], 0) = best;
            *cluster.map_shared_rank(&cand_i[rank], 0) = idx;
        }
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        best = cand_v[0];
        idx = cand_i[0];
        for (int c = 1; c < ranks; ++c) argmax_merge(best, idx, cand_v[c], cand_i[c]);
        out[blockIdx.y] = idx < V ? idx : 0;
    }
}

// grid (ranks, rows), clusters of `ranks` blocks along x; V <= ranks * kChunkFloats.
// Each block keeps its chunk of the row in shared memory: read once from global
// memory as logits / T, rewritten as exp(. - max) once the cluster's maximum is
// known.  Every thread owns a contiguous segment of the chunk, so cumulative sums
// run in vocabulary order: segments within a warp by a prefix scan, warps and
// blocks in order.  The block, warp and segment that hold the target u * total are
// found by comparing it with these same partial sums, and the owner of the segment
// walks it.  Should rounding leave the target at or beyond the total, the last
// entry of non-zero probability is taken.
__global__ void __launch_bounds__(kRowThreads)
sample_temperature_cluster_kernel(const float* __restrict__ logits, int ld, int V, float inv_temperature,
                                  unsigned long long seed, const int* __restrict__ sequence_ids,
                                  const int* __restrict__ steps, int* __restrict__ out) {
    chain_release();
    chain_wait();
    extern __shared__ float vals[];                       // the chunk
    __shared__ float wred[kRowThreads / 32];
    __shared__ float cmax[kMaxRanks], ctot[kMaxRanks];
    __shared__ int clast[kMaxRanks];                      // each block's last entry of non-zero probability, or -1
    __shared__ int wlast[kRowThreads / 32];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), ranks = (int)cluster.num_blocks();
    const int r = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* row = logits + (size_t)r * ld;
    const int chunk = row_chunk(V, ranks);
    const int begin = min(V, rank * chunk), n = min(V, begin + chunk) - begin;

    // ---- the chunk into shared memory, and its maximum
    float mx = -INFINITY;
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int n4 = vec ? n / 4 : 0;
    {
        const float4* src = reinterpret_cast<const float4*>(row + begin);
        int i = tid;
        for (; i + 3 * kRowThreads < n4; i += 4 * kRowThreads) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = src[i + u * kRowThreads];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 z = make_float4(v[u].x * inv_temperature, v[u].y * inv_temperature,
                                             v[u].z * inv_temperature, v[u].w * inv_temperature);
                reinterpret_cast<float4*>(vals)[i + u * kRowThreads] = z;
                mx = fmaxf(fmaxf(mx, fmaxf(z.x, z.y)), fmaxf(z.z, z.w));
            }
        }
        for (; i < n4; i += kRowThreads) {
            const float4 v = src[i];
            const float4 z = make_float4(v.x * inv_temperature, v.y * inv_temperature,
                                         v.z * inv_temperature, v.w * inv_temperature);
            reinterpret_cast<float4*>(vals)[i] = z;
            mx = fmaxf(fmaxf(mx, fmaxf(z.x, z.y)), fmaxf(z.z, z.w));
        }
        for (int k = 4 * n4 + tid; k < n; k += kRowThreads) {
            const float z = row[begin + k] * inv_temperature;
            vals[k] = z;
            mx = fmaxf(mx, z);
        }
    }
    mx = warp_max(mx);
    if (lane == 0) wred[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        mx = wred[0];
        for (int w = 1; w < kRowThreads / 32; ++w) mx = fmaxf(mx, wred[w]);
        for (int c = 0; c < ranks; ++c) *cluster.map_shared_rank(&cmax[rank], c) = mx;
    }
    cluster.sync();
    mx = cmax[0];
    for (int c = 1; c < ranks; ++c) mx = fmaxf(mx, cmax[c]);

    // ---- exp(z - max) in place; this thread's segment sum, and where its last non-zero entry is
    const int seg = ((n + kRowThreads - 1) / kRowThreads) | 1;   // odd: neighbouring threads fall in different banks
    const int s_begin = min(n, tid * seg), s_end = min(n, s_begin + seg);
    float s = 0.f;
    int last = -1;
    for (int k = s_begin; k < s_end; ++k) {
        const float e = expf(vals[k] - mx);
        vals[k] = e;
        s += e;
        if (e > 0.f) last = begin + k;
    }
    // inclusive prefix over the warp's segments, in lane order
    float incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    int wl = last;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wl = max(wl, __shfl_xor_sync(0xffffffffu, wl, o));
    __syncthreads();                                      // wred is read above by thread 0
    if (lane == 31) wred[warp] = incl;                    // the warp's total
    if (lane == 0) wlast[warp] = wl;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.f;
        int bl = -1;
        for (int w = 0; w < kRowThreads / 32; ++w) { tot += wred[w]; bl = max(bl, wlast[w]); }
        for (int c = 0; c < ranks; ++c) {
            *cluster.map_shared_rank(&ctot[rank], c) = tot;
            *cluster.map_shared_rank(&clast[rank], c) = bl;
        }
    }
    cluster.sync();

    // ---- which block, warp and segment hold the target
    float total = 0.f;
    for (int c = 0; c < ranks; ++c) total += ctot[c];
    const float target = uniform24(seed, sequence_ids[r], steps[r]) * total;
    float before = 0.f;                                   // cumulative sum ahead of this block
    int owner = -1;
    {
        float run = 0.f;
        for (int c = 0; c < ranks; ++c) {
            if (c == rank) before = run;
            if (owner < 0 && target < run + ctot[c]) owner = c;
            run += ctot[c];
        }
    }
    if (owner < 0) {                                      // rounding: the last entry that can be drawn at all
        if (rank == 0 && tid == 0) {
            int bl = 0;
            for (int c = 0; c < ranks; ++c) bl = max(bl, clast[c]);
            out[r] = bl;
        }
        return;
    }
    if (owner != rank) return;
    float wbefore = before;                               // ahead of this warp
    int wown = -1;
    {
        float run = before;
        for (int w = 0; w < kRowThreads / 32; ++w) {
            if (w == warp) wbefore = run;
            if (wown < 0 && target < run + wred[w]) wown = w;
            run += wred[w];
        }
    }
    if (wown < 0) {                                       // the block's sum said yes, the warps' running sums no
        if (tid == 0) out[r] = max(clast[rank], 0);
        return;
    }
    if (wown != warp) return;
    // the first lane whose inclusive sum passes the target
    const bool mine_passes = target < wbefore + incl;
    const unsigned passes = __ballot_sync(0xffffffffu, mine_passes);
    if (passes == 0u) {
        if (lane == 0) out[r] = max(wlast[warp], 0);
        return;
    }
    if (lane != __ffs(passes) - 1) return;
    float c = wbefore + (incl - s);
    int pick = -1;
    for (int k = s_begin; k < s_end; ++k) {
        c += vals[k];
        if (c > target) { pick = begin + k; break; }
    }
    out[r] = pick >= 0 ? pick : max(last, 0);
}
}  // namespace

GTG_API int gtg_argmax(const float* logits, int ld, int R, int V, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return kErrBadArgument;
    if (V >= 8192 && R <= 65535)
        return launch_chained_cluster(argmax_cluster_kernel, dim3(row_ranks(V, 8192), R), dim3(kRowThreads),
                                      row_ranks(V, 8192), 0, stream, logits, ld, V, out);
    return launch_chained(argmax_kernel, dim3(R), dim3(kArgmaxThreads), 0, stream, logits, ld, V, out);
}

GTG_API int gtg_sample_temperature(const float* logits, int ld, int R, int V, float temperature,
                                   unsigned long long seed, const int* sequence_ids,
                                   const int* steps, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V || !(temperature > 0.f)) return kErrBadArgument;
    if (V >= 4096 && V <= kMaxRanks * kChunkFloats && R <= 65535) {
        const int ranks = row_ranks(V, kChunkFloats);
        const size_t smem = (size_t)(((V + ranks - 1) / ranks + 3) / 4 * 4) * sizeof(float);
        static size_t configured = 0;
        if (smem > configured) {
            const cudaError_t e = cudaFuncSetAttribute(sample_temperature_cluster_kernel,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = smem;
        }
        return launch_chained_cluster(sample_temperature_cluster_kernel, dim3(ranks, R), dim3(kRowThreads), ranks,
                                      smem, stream, logits, ld, V, 1.0f / temperature, seed, sequence_ids, steps, out);
    }
    return launch_chained(sample_temperature_kernel, dim3(R), dim3(kThreads), 0, stream, logits, ld, V,
                          1.0f / temperature, seed, sequence_ids, steps, out);
}

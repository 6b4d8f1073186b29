// Shared helpers of the sm_100a kernels: value conversion, warp and block
// reductions, the page geometry of the key/value cache, and launch checking.
// Every launcher is an `extern "C"` function that takes raw device pointers and
// the stream to launch on, and returns a cudaError_t as int (0 = success).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define GTG_API extern "C" __attribute__((visibility("default")))

// Tokens per cache page.  A request's cache footprint is its token count rounded
// up to a multiple of this.
constexpr int kPageTokens = 64;

// Error codes beyond cudaError_t returned by launchers (negative, so they never
// collide with CUDA's).
constexpr int kErrBadArgument = -1;
constexpr int kErrUnsupported = -2;

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Layout of the key/value cache of one cache entry (one run of one layer).
// A page holds kPageTokens tokens of every key/value head:
//   page p, head h, token t, channel d -> base + p*page_stride + (h*kPageTokens + t)*head_dim + d
// Keys and values have separate bases and share page indices.
// `block_table[slot*table_stride + i]` is the page that holds tokens
// [i*64, i*64+64) of the sequence in `slot`.
struct KVPages {
    void* k;
    void* v;
    long long page_stride;   // elements between consecutive pages
    const int* block_table;
    int table_stride;        // entries per slot
};

static inline int launch_status() {
    return (int)cudaGetLastError();
}

// ---- programmatic dependent launch -------------------------------------------
// A kernel launched through launch_chained() may begin while the kernels before it
// in the stream are still running: its blocks become resident and run up to
// chain_wait(), which returns once the kernel before it has completed and its
// writes are visible.  Before chain_wait() a kernel may only do work that depends
// on nothing a previous kernel wrote (index arithmetic, barrier set-up, copies of
// weights).  chain_release() lets the kernel after this one begin in the same
// way.  The weight-streaming products issue it after chain_wait(); the small
// kernels between them (norms, rotation, merges, sampling) issue it first, so
// that the next product's blocks can move in beside the previous product's last
// blocks and start their weight copies while it drains.  Completion is still
// ordered: every kernel waits for its predecessor, which waited for its own.
// Launched without the attribute (the switch off, or a plain <<<>>> launch) both
// are no-ops.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// One switch per compiled library (each .cu file is its own library).
static int g_chained_launch = 0;
GTG_API void gtg_set_chained_launch(int on) { g_chained_launch = on ? 1 : 0; }

template <typename... Params, typename... Args>
static inline int launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_chained_launch ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
    return e != cudaSuccess ? (int)e : launch_status();
}

// The same for a grid of thread-block clusters of `cluster_x` blocks along x.
template <typename... Params, typename... Args>
static inline int launch_chained_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, int cluster_x,
                                         size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_chained_launch ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
    return e != cudaSuccess ? (int)e : launch_status();
}

// The allocation-free variant of split-KV decode attention declared in
// attention_decode_static.h.  It reuses the kernels of attention_bf16.cu (that
// file is compiled into this library as well, unchanged) and differs only in
// where the partial results of the splits live: a file-scope device array
// instead of a buffer from the caller.
#include "attention_bf16.cu"
#include "attention_decode_static.h"

#include <mutex>

namespace {

// The scratch itself.  In host code this name is only a stand-in for the
// symbol; its device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_static_scratch[GTG_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_address[kMaxDevices] = {};
std::mutex g_setup_lock;

// Device address of the array on the current device; looked up once per device.
int static_scratch(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return kErrUnsupported;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (g_scratch_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return kErrBadArgument;
        g_scratch_address[dev] = p;
    }
    *out = g_scratch_address[dev];
    return 0;
}
}  // namespace

GTG_API long long gtg_static_scratch_capacity_floats(void) { return GTG_STATIC_SCRATCH_FLOATS; }

GTG_API int gtg_attention_decode_bf16_static(const void* q, int ldq, void* out, int ldo,
                                             const void* kc, const void* vc, long long page_stride,
                                             const int* block_table, int table_stride,
                                             const int* slots, const int* positions,
                                             int n_seqs, int n_heads, int n_kv, int head_dim,
                                             float scale, int window, int n_splits,
                                             cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_splits < 1) return kErrBadArgument;
    const long long need = gtg_attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits);
    if (need > GTG_STATIC_SCRATCH_FLOATS) return GTG_ERR_STATIC_SCRATCH_TOO_SMALL;
    float* scratch = nullptr;
    if (n_splits > 1) {
        const int st = static_scratch(&scratch);
        if (st != 0) return st;
    }
    return gtg_attention_decode_bf16(q, ldq, out, ldo, kc, vc, page_stride, block_table, table_stride,
                                     slots, positions, n_seqs, n_heads, n_kv, head_dim, scale, window,
                                     n_splits, scratch, 0, 0, stream);
}

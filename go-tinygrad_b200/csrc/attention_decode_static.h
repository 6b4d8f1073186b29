// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project: it exists for
// users of this library whose code runs where cudaMalloc is not available to
// them -- a plugin inside a host application that owns the allocator and hands
// out only input and output buffers, a real-time loop that forbids allocation
// after start-up, or a process whose memory budget was fixed by someone else.
// The regular entry point (gtg_attention_decode_bf16) asks the caller for a
// scratch buffer when the keys of a sequence are split over several thread
// blocks; this one keeps that scratch in a fixed array inside the library.
//
// What to know before using it:
//   * The array holds GTG_STATIC_SCRATCH_FLOATS floats (4 MiB).  It is part of the
//     loaded library image: every GPU whose context loads the library holds
//     those 4 MiB until the process exits, whether or not this function is
//     ever called.
//   * A call that would need more scratch than that is refused with
//     GTG_ERR_STATIC_SCRATCH_TOO_SMALL and launches nothing.  The need is
//     sequences * query_heads * n_splits * (padded_head_dim + 2) floats for
//     n_splits > 1 and zero for n_splits == 1
//     (gtg_attention_decode_scratch_floats computes it).
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make
//     that first call outside of any stream capture.
//   * All calls share the one array and it keeps the previous call's contents.
//     Nothing has to be cleared: each call writes every element it later reads.
//     Two calls that overlap on the GPU (different streams, or the same graph
//     replayed concurrently) race on it; keep calls on one stream or order them
//     yourself.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats.
#define GTG_STATIC_SCRATCH_FLOATS (1 << 20)

// Returned (and nothing is launched) when the call needs more scratch than the
// built-in array holds.
#define GTG_ERR_STATIC_SCRATCH_TOO_SMALL (-3)

// Same arguments and result as gtg_attention_decode_bf16, without the scratch
// pointer.  Returns 0 on success, a negative library code or a cudaError_t.
int gtg_attention_decode_bf16_static(const void* q, int ldq, void* out, int ldo,
                                     const void* kc, const void* vc, long long page_stride,
                                     const int* block_table, int table_stride,
                                     const int* slots, const int* positions,
                                     int n_seqs, int n_heads, int n_kv, int head_dim,
                                     float scale, int window, int n_splits, cudaStream_t stream);

// GTG_STATIC_SCRATCH_FLOATS, for callers that bind the symbol at run time.
long long gtg_static_scratch_capacity_floats(void);

#ifdef __cplusplus
}
#endif

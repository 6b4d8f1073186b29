// Weight-streaming bfloat16 product for decode steps: C[M,N] = X[M,K] . W[N,K]^T
// with few rows M (one token per live sequence, M <= 64).  The work is reading W
// once from HBM; everything is shaped around that.
//
//   * A tile of 16 output features (rows of W) is the M dimension of
//     mma.sync.m16n8k16, the tokens are its N dimension (8 per tile).
//   * A CTA's 8 warps split K: warp w takes the 32-wide k blocks w, w+8, ...  Each
//     thread loads 16 bytes (8 consecutive k) of rows g and g+8; the MMA's k slots are
//     assigned to those 8 values in the order they lie in memory (a dot product does
//     not care about the order of k as long as both operands agree), so no shuffle or
//     shared-memory transposition is needed.
//   * Two forms.  The persistent one (gemm_stream_kernel, up to 16 tokens, K a
//     multiple of 64; described above its code) keeps two CTAs on every SM, each with
//     a ring of three 32 KB pieces of W that arrive by one tensor copy (TMA) each.
//     The other (gemm_skinny_kernel: any K that is a multiple of 8, up to 64 tokens)
//     gives every 16-row tile a CTA of its own, whose 16 rows of up to 2048 values
//     arrive by sixteen bulk copies on one mbarrier.
//   * Rows longer than 2048 values are split over a thread-block cluster (2 to 8 CTAs
//     along k) whose partial sums meet through the cluster's shared memory, so that a
//     product with few output features and a long inner size still fills the GPU.
//   * Every wait on an mbarrier is bounded: if the copies never land, the kernel
//     records it in a status word (gtg_gemm_bf16_skinny_status) and returns.
//   * X stays in L1/L2 (read by every CTA) and is loaded with plain loads.
//   * Partial sums are added in a fixed order (warps, then cluster ranks): the
//     result does not depend on timing.
// Any N; output bfloat16 or float.
#include "mma_helpers.cuh"
#include <cooperative_groups.h>
#include <cuda.h>

namespace cg = cooperative_groups;

namespace {
constexpr int kWarps = 8;
constexpr int kBlocksPerWarp = 8;                       // k blocks of 32 per warp and pass
constexpr int kPassK = kWarps * kBlocksPerWarp * 32;    // 2048 values of k per CTA and pass
constexpr int kMaxCluster = 8;

constexpr int kRowPad = 64;                              // bytes between rows of the staged tile
constexpr int kRowStride = kPassK * 2 + kRowPad;
constexpr int kTileBytes = 16 * kRowStride;
constexpr unsigned kSpinLimit = 1u << 22;
// The kernels of this library exist twice: as they run, and (kTest) in the form the
// test of the give-up path launches, whose waits poll a thousand times instead of
// millions and whose asynchronous copies are not issued at all, so that every
// barrier it waits on never completes.  The second form is the first form's code
// with these two constants changed; see the test hook at the end of this file.
template <bool kTest> struct Waits {
    static constexpr unsigned kLimit = kTest ? 1024u : kSpinLimit;
    static constexpr bool kSkipCopies = kTest;
};
static bool g_test_waits = false;       // set by the test hook: launches take the kTest form


__device__ int g_status = 0;                             // 1: a wait on the copies gave up

__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
template <bool kTest>
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    if (Waits<kTest>::kSkipCopies) return;
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// True once the phase with this parity has completed; gives up after kSpinLimit polls.
template <bool kTest>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned i = 0; i < Waits<kTest>::kLimit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                     "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// Writes one output of a 16-feature tile; every lane of the warp must call it.
//   epi == 0: C[m][n0 + r] = s.
//   epi == 1: SwiGLU over a tile that holds 8 gate features followed by their 8
//             up features: the thread of gate r < 8 fetches the up value from the
//             thread of r + 8 and writes silu(gate) * up to C[m][n0/2 + r].
template <typename OutT>
__device__ __forceinline__ void store_feature(OutT* C, int ldc, int m, int n0, int r, int M, int N,
                                              float s, int epi) {
    if (epi == 0) {
        if (m < M && n0 + r < N) C[(size_t)m * ldc + n0 + r] = from_f32<OutT>(s);
        return;
    }
    const float up = __shfl_down_sync(0xffffffffu, s, 8);
    if (r < 8 && m < M && n0 + r + 8 < N)
        C[(size_t)m * ldc + (n0 >> 1) + r] = from_f32<OutT>(s / (1.0f + expf(-s)) * up);
}

// grid = (ceil(N/16), S) with clusters of (1, S, 1): blockIdx.y is the CTA's
// rank in its cluster and the index of its slice [rank*k_slice, +k_slice) of k.
template <int NT, typename OutT, bool kTest>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(const bf16* __restrict__ X, int ldx, const bf16* __restrict__ W, int ldw,
                   OutT* __restrict__ C, int ldc, int M, int N, int K, int k_slice, int epi) {
    extern __shared__ __align__(128) unsigned char tile[];      // 16 rows of W, kRowStride apart
    __shared__ float red[kWarps][16][NT * 8 + 1];        // later reused for the cluster's partial sums
    __shared__ __align__(8) unsigned long long bar_storage;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int rank = blockIdx.y, n_ranks = gridDim.y;
    const int k_begin = rank * k_slice, k_end = min(K, k_begin + k_slice);
    const uint32_t bar = smem_u32(&bar_storage), tile_addr = smem_u32(tile);
    if (threadIdx.x == 0) mbar_init(bar, 1);
    __syncthreads();
    chain_wait();
    chain_release();
    const bf16* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) xrow[j] = X + (size_t)min(j * 8 + g, M - 1) * ldx + t * 8;

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

    uint32_t parity = 0;
    for (int base = k_begin; base < k_end; base += kPassK) {
        const int k_len = min(kPassK, k_end - base);          // a multiple of 8
        if (threadIdx.x == 0) {
            mbar_expect_tx(bar, 16u * (uint32_t)k_len * 2u);
            for (int r = 0; r < 16; ++r)                       // rows beyond N repeat the last one; dropped at the store
                bulk_copy<kTest>(tile_addr + r * kRowStride, W + (size_t)min(n0 + r, N - 1) * ldw + base,
                          (uint32_t)k_len * 2u, bar);
        }
        // The CTA decides as one whether the copies arrived (a block barrier ends every
        // pass, so its threads may not part ways here).  If a wait gave up: say so and
        // stop copying -- a barrier whose phase never completed must not be armed again
        // -- but stay for the sums and the cluster barriers below, where the peers of a
        // cluster wait; the status word tells the host that the result is void.
        if (__syncthreads_or(!mbar_wait<kTest>(bar, parity))) {
            if (threadIdx.x == 0) atomicExch(&g_status, 1);
            break;
        }
        parity ^= 1;
#pragma unroll
        for (int u = 0; u < kBlocksPerWarp; ++u) {
            const int kl = (warp + u * kWarps) * 32 + t * 8;   // this thread's 8 values of k within the pass
            const bool ok = kl < k_len;
            uint4 wa = make_uint4(0, 0, 0, 0), wb = wa;
            if (ok) {
                wa = *reinterpret_cast<const uint4*>(tile + g * kRowStride + kl * 2);
                wb = *reinterpret_cast<const uint4*>(tile + (g + 8) * kRowStride + kl * 2);
            }
            const uint32_t a_lo[4] = {wa.x, wb.x, wa.y, wb.y};
            const uint32_t a_hi[4] = {wa.z, wb.z, wa.w, wb.w};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 xb = ok ? ld_cached16(xrow[j] + base + kl - t * 8) : make_uint4(0, 0, 0, 0);
                mma_bf16_16816(acc[j], a_lo, xb.x, xb.y);
                mma_bf16_16816(acc[j], a_hi, xb.z, xb.w);
            }
        }
        __syncthreads();                                       // the tile is free for the next pass
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
    if (n_ranks == 1) {
        for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kWarps * 32) {
            const int m = idx >> 4, r = idx & 15;          // consecutive threads -> consecutive features
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[w][r][m];
            store_feature<OutT>(C, ldc, m, n0, r, M, N, s, epi);
        }
        return;
    }
    // Several CTAs share the rows.  Every rank sums its warps into registers; once
    // all ranks have done so (first cluster barrier) rank 0's `red` is free and
    // receives one block of sums per rank; after the second barrier rank 0 adds
    // them in rank order.
    constexpr int kPerThread = (16 * NT * 8 + kWarps * 32 - 1) / (kWarps * 32);
    float mine[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
        const int idx = threadIdx.x + i * kWarps * 32;
        float s = 0.f;
        if (idx < 16 * NT * 8) {
            const int m = idx >> 4, r = idx & 15;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) s += red[w][r][m];
        }
        mine[i] = s;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    float* gather = cluster.map_shared_rank(&red[0][0][0], 0);     // [rank][16 * NT * 8] in rank 0
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
        const int idx = threadIdx.x + i * kWarps * 32;
        if (idx < 16 * NT * 8) gather[rank * 16 * NT * 8 + idx] = mine[i];
    }
    cluster.sync();
    if (rank != 0) return;
    const float* sums = &red[0][0][0];
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += kWarps * 32) {
        const int m = idx >> 4, r = idx & 15;
        float s = 0.f;
        for (int c = 0; c < n_ranks; ++c) s += sums[c * 16 * NT * 8 + idx];
        store_feature<OutT>(C, ldc, m, n0, r, M, N, s, epi);
    }
}

template <int NT, typename OutT, bool kTest = false>
int launch_typed(const bf16* X, int ldx, const bf16* W, int ldw, OutT* C, int ldc,
                 int M, int N, int K, int epi, cudaStream_t stream) {
    // the fewest ranks (a power of two, at most 8) whose slice fits one pass
    int ranks = 1;
    while (ranks < kMaxCluster && (K + ranks - 1) / ranks > kPassK) ranks *= 2;
    const int k_slice = (((K + ranks - 1) / ranks) + 31) / 32 * 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + 15) / 16, ranks, 1);
    cfg.blockDim = dim3(kWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = kTileBytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t ce = cudaFuncSetAttribute(gemm_skinny_kernel<NT, OutT, kTest>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes);
        if (ce != cudaSuccess) return (int)ce;
        configured = true;
    }
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ranks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_chained_launch ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<NT, OutT, kTest>, X, ldx, W, ldw, C, ldc, M, N, K, k_slice, epi);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// ---------------------------------------------------------------- persistent form
// For M <= 16, K <= 16384 and K a multiple of 64.  The grid is one cluster-row of
// CTAs per SM-sized share of the GPU; CTA (c, rank) walks the row tiles c, c+G,
// c+2G, ... of its slice of k.  A row tile arrives as one or two pieces of 1024
// values of k, each by ONE tensor copy (TMA) through a ring of three staged
// pieces: while a piece is multiplied, two more are in flight.  W is described to
// the copy engine as [k/64][row][64 values] (the middle stride is the row pitch),
// so a piece lands as sixteen blocks of 16 rows x 128 bytes with the 128-byte
// swizzle, and the 16-byte fragment reads of rows g and g+1 fall in different
// banks without padding.  The ring and the sums take half of an SM's shared
// memory, so two CTAs share an SM (six pieces, 192 KB, in flight per SM: what the
// kernel reaches is set by that figure over the latency of a copy), and under
// programmatic dependent launch a CTA of the next product of the step moves in as
// soon as one of these leaves and fills its own ring while this product drains,
// so the memory system stays busy across the boundary between kernels.  The
// activations of the slice are the same for every row tile, so each thread loads
// its fragments of X once, into registers.
constexpr int kPieceK = 1024;                            // values of k per staged piece
constexpr int kPieceBlocks = kPieceK / (kWarps * 32);    // k blocks of 32 per warp and piece
constexpr int kPieceBytes = 16 * kPieceK * 2;
constexpr int kRing = 3;

template <bool kTest>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    if (Waits<kTest>::kSkipCopies) return;
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int NT, typename OutT, bool kTest>
__global__ void __launch_bounds__(kWarps * 32, 2)
gemm_stream_kernel(const bf16* __restrict__ X, int ldx, const __grid_constant__ CUtensorMap map_w,
                   OutT* __restrict__ C, int ldc, int M, int N, int K, int k_slice, int epi) {
    extern __shared__ __align__(1024) unsigned char ring_raw[];
    constexpr int kSlot = 16 * NT * 8;                          // sums of one row tile
    constexpr int kSlots = kWarps * 16 * (NT * 8 + 1) / kSlot;  // 9 (NT = 1) or 8 that `red` holds
    constexpr int kBatchMax = NT == 1 ? 8 : 7;                  // what fits beside the ring with two CTAs per SM
    __shared__ float red[kWarps][16][NT * 8 + 1];               // also receives the cluster's partial sums
    __shared__ float pending[kBatchMax * kSlot];                // this rank's sums of a batch of row tiles
    __shared__ __align__(8) unsigned long long bar_storage[kRing];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rank = blockIdx.y, n_ranks = gridDim.y;
    const int k_begin = rank * k_slice, k_len = min(K, k_begin + k_slice) - k_begin;   // k_len <= kPassK
    const int row_tiles = (N + 15) / 16;
    const int n_pieces = k_len > kPieceK ? 2 : 1;               // pieces per row tile
    const int my_tiles = (int)blockIdx.x < row_tiles ? (row_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int n_items = my_tiles * n_pieces;
    const uint32_t bar0 = smem_u32(&bar_storage[0]);
    const uint32_t ring0 = (smem_u32(ring_raw) + 1023u) & ~1023u;   // the swizzle pattern repeats every 1024 bytes
    const unsigned char* ring = ring_raw + (ring0 - smem_u32(ring_raw));
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRing; ++s) mbar_init(bar0 + 8 * s, 1);
    }
    __syncthreads();

    auto issue = [&](int item) {                                // thread 0 only
        const int stage = item % kRing;
        const int tile = blockIdx.x + (item / n_pieces) * gridDim.x, piece = item % n_pieces;
        const uint32_t bar = bar0 + 8 * stage;
        mbar_expect_tx(bar, (uint32_t)kPieceBytes);             // rows beyond N and blocks beyond K arrive as zeros
        tma_load_3d<kTest>(ring0 + stage * kPieceBytes, &map_w, 0, tile * 16, (k_begin + piece * kPieceK) / 64, bar);
    };
    if (threadIdx.x == 0) {
        for (int item = 0; item < kRing && item < n_items; ++item) issue(item);
    }

    // The weights depend on no earlier kernel, so their first copies are already in
    // flight; the activations do.
    chain_wait();
    chain_release();

    // this thread's fragments of the activations: 8 k blocks x NT token tiles
    uint4 xf[2 * kPieceBlocks][NT];
    bool ok[2 * kPieceBlocks];
#pragma unroll
    for (int u = 0; u < 2 * kPieceBlocks; ++u) {
        const int kl = (u / kPieceBlocks) * kPieceK + (warp + (u % kPieceBlocks) * kWarps) * 32 + t * 8;
        ok[u] = kl < k_len;                                     // beyond it the piece holds a neighbour's k or zeros
#pragma unroll
        for (int j = 0; j < NT; ++j)
            xf[u][j] = ok[u] ? ld_cached16(X + (size_t)min(j * 8 + g, M - 1) * ldx + k_begin + kl)
                             : make_uint4(0, 0, 0, 0);
    }

    cg::cluster_group cluster = cg::this_cluster();
    // row tiles per exchange: ceil(batch / ranks) * ranks slots must fit into `red`
    const int batch = min(kBatchMax, (min(kSlots, 8) / n_ranks) * n_ranks);
    bool failed = false;
    float acc[NT][4];
    for (int item = 0; item < n_items; ++item) {
        const int stage = item % kRing, piece = item % n_pieces;
        // A wait that gives up ends all waiting and all copying of this CTA (a barrier whose
        // phase never completed must not be armed again), but not its walk through the
        // tiles: its peers wait for it at the cluster barriers below.
        if (!failed && !mbar_wait<kTest>(bar0 + 8 * stage, (uint32_t)(item / kRing) & 1u)) failed = true;
        const unsigned char* tl = ring + stage * kPieceBytes;
        if (piece == 0) {
#pragma unroll
            for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
        }
        auto multiply = [&](int first) {
#pragma unroll
            for (int v = 0; v < kPieceBlocks; ++v) {
                const int u = first + v;
                const int blk32 = warp + v * kWarps;                       // 32 values of k: half of a 64-value block
                // block [blk32/2] of 16 rows x 128 bytes; 16-byte chunk (blk32&1)*4 + t of row g, swizzled by the row
                const unsigned char* at = tl + (blk32 >> 1) * 2048 + g * 128 + (((((blk32 & 1) << 2) | t) ^ (g & 7)) << 4);
                uint4 wa = make_uint4(0, 0, 0, 0), wb = wa;
                if (ok[u] && !failed) {
                    wa = *reinterpret_cast<const uint4*>(at);
                    wb = *reinterpret_cast<const uint4*>(at + 8 * 128);   // row g + 8: the same swizzle
                }
                const uint32_t a_lo[4] = {wa.x, wb.x, wa.y, wb.y};
                const uint32_t a_hi[4] = {wa.z, wb.z, wa.w, wb.w};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    mma_bf16_16816(acc[j], a_lo, xf[u][j].x, xf[u][j].y);
                    mma_bf16_16816(acc[j], a_hi, xf[u][j].z, xf[u][j].w);
                }
            }
        };
        if (piece == 0) multiply(0); else multiply(kPieceBlocks);   // register indices stay constant
        __syncthreads();                                            // the piece has been read: its stage is free,
        if (threadIdx.x == 0 && !failed && item + kRing < n_items) issue(item + kRing);   // and so is `red` (read before this barrier)
        if (piece != n_pieces - 1) continue;
        const int tile_no = item / n_pieces;                        // among this CTA's row tiles
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            red[warp][g][j * 8 + t * 2] = acc[j][0];
            red[warp][g][j * 8 + t * 2 + 1] = acc[j][1];
            red[warp][g + 8][j * 8 + t * 2] = acc[j][2];
            red[warp][g + 8][j * 8 + t * 2 + 1] = acc[j][3];
        }
        __syncthreads();
        // 16 features x NT*8 tokens: at most one sum per thread (NT <= 2)
        const int idx = threadIdx.x, m = idx >> 4, r = idx & 15;
        const bool mine_valid = idx < kSlot;
        float mine = 0.f;
        if (mine_valid) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mine += red[w][r][m];
        }
        if (n_ranks == 1) {
            if (mine_valid)                                       // uniform per warp: whole warps are valid or not
                store_feature<OutT>(C, ldc, m, (blockIdx.x + tile_no * gridDim.x) * 16, r, M, N, mine, epi);
            continue;
        }
        // The ranks' sums of a row tile meet through shared memory of the cluster, a batch
        // of row tiles at a time (two cluster barriers per batch, not per tile): tile i of
        // the batch is summed and written by rank i % ranks, which receives the others'
        // sums for it in its own `red`, in slot (i / ranks) * ranks + sender.
        const int in_batch = tile_no % batch;
        if (mine_valid) pending[in_batch * kSlot + idx] = mine;
        if (in_batch != batch - 1 && tile_no != my_tiles - 1) continue;
        const int n_batch = in_batch + 1, first = tile_no - in_batch;
        cluster.sync();                                           // every rank is done with its own `red`
        for (int i = 0; i < n_batch; ++i) {
            float* dst = cluster.map_shared_rank(&red[0][0][0], i % n_ranks);
            if (mine_valid) dst[((i / n_ranks) * n_ranks + rank) * kSlot + idx] = pending[i * kSlot + idx];
        }
        cluster.sync();
        for (int i = rank; i < n_batch; i += n_ranks) {
            const float* sums = &red[0][0][0] + (i / n_ranks) * n_ranks * kSlot;
            float total = 0.f;
            if (mine_valid) {
                for (int c = 0; c < n_ranks; ++c) total += sums[c * kSlot + idx];
                store_feature<OutT>(C, ldc, m, (blockIdx.x + (first + i) * gridDim.x) * 16, r, M, N, total, epi);
            }
        }
        // the next tile writes `red` only after the barrier that follows its multiplication
    }
    if (failed && threadIdx.x == 0) atomicExch(&g_status, 1);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

// W[N, K] (row pitch ldw) as [K/64][N][64]: boxes of 16 blocks x 16 rows x 64 values.
bool stream_map(CUtensorMap* map, const bf16* W, int ldw, int N, int K) {
    EncodeTiled enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[3] = {64, (cuuint64_t)N, (cuuint64_t)(K / 64)};
    const cuuint64_t strides[2] = {(cuuint64_t)ldw * 2, 128};
    const cuuint32_t box[3] = {64, 16, kPieceK / 64};
    const cuuint32_t elem[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16*>(W), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// kErrUnsupported when this form does not serve the sizes (the caller then takes the other one).
template <int NT, typename OutT, bool kTest = false>
int launch_stream(const bf16* X, int ldx, const bf16* W, int ldw, OutT* C, int ldc,
                  int M, int N, int K, int epi, cudaStream_t stream) {
    if (K % 64) return kErrUnsupported;
    const int row_tiles = (N + 15) / 16;
    int ranks = (K + kPassK - 1) / kPassK;      // whole passes where K allows: no piece is copied half empty
    if (ranks > kMaxCluster) return kErrUnsupported;
    // few rows: split k further (down to one piece per rank) until every SM has two blocks to run
    while (2 * ranks <= kMaxCluster && row_tiles * ranks < 2 * 148 && (K + 2 * ranks - 1) / (2 * ranks) >= kPieceK) ranks *= 2;
    const int k_slice = (((K + ranks - 1) / ranks) + 63) / 64 * 64;
    if (k_slice > kPassK) return kErrUnsupported;
    CUtensorMap map_w;
    if (!stream_map(&map_w, W, ldw, N, K)) return kErrUnsupported;
    const int smem = kRing * kPieceBytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t ce = cudaFuncSetAttribute(gemm_stream_kernel<NT, OutT, kTest>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (ce != cudaSuccess) return (int)ce;
        configured = true;
    }
    int per_rank = 2 * 148 / ranks;             // two CTAs per SM: six pieces in flight; a finished CTA makes room for the next kernel
    if (per_rank < 1) per_rank = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(row_tiles < per_rank ? row_tiles : per_rank, ranks, 1);
    cfg.blockDim = dim3(kWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ranks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // A cluster needs all its CTAs in one GPC, so fewer clusters can be resident than
    // 2 * SMs / ranks says; a grid beyond that runs its last clusters as a second wave.
    // The count the runtime gives holds for an empty GPU.  These clusters arrive while
    // the blocks of the product before are still leaving, take the places that happen
    // to be free, and then pack less well: clusters of three and more get a twelfth
    // fewer (measured: of 71 clusters of four and of 37 of seven some came late).
    static int resident[kMaxCluster + 1] = {};
    if (ranks > 1 && resident[ranks] == 0) {
        int n = 0;
        resident[ranks] = cudaOccupancyMaxActiveClusters(&n, gemm_stream_kernel<NT, OutT, kTest>, &cfg) == cudaSuccess && n > 0
                              ? n : -1;
        cudaGetLastError();
        if (ranks > 2 && resident[ranks] > 12) resident[ranks] -= (resident[ranks] + 11) / 12;
    }
    if (ranks > 1 && resident[ranks] > 0 && (int)cfg.gridDim.x > resident[ranks]) {
        // the fewest clusters that still finish in as many rounds of row tiles
        const int rounds = (row_tiles + resident[ranks] - 1) / resident[ranks];
        cfg.gridDim.x = (row_tiles + rounds - 1) / rounds;
    }
    cfg.numAttrs = g_chained_launch ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NT, OutT, kTest>, X, ldx, map_w, C, ldc, M, N, K, k_slice, epi);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

template <int NT>
int launch(const bf16* X, int ldx, const bf16* W, int ldw, void* C, int ldc, int out_f32,
           int M, int N, int K, int epi, cudaStream_t stream) {
    if (g_test_waits) {                        // the give-up test: bfloat16 results of up to 16 rows
        if constexpr (NT <= 2) {
            if (out_f32) return kErrUnsupported;
            if (K <= kMaxCluster * kPassK) {
                const int st = launch_stream<NT, bf16, true>(X, ldx, W, ldw, (bf16*)C, ldc, M, N, K, epi, stream);
                if (st != kErrUnsupported) return st;
            }
            return launch_typed<NT, bf16, true>(X, ldx, W, ldw, (bf16*)C, ldc, M, N, K, epi, stream);
        }
        return kErrUnsupported;
    }
    if constexpr (NT <= 2) {
        if (K <= kMaxCluster * kPassK) {
            const int st = out_f32 ? launch_stream<NT, float>(X, ldx, W, ldw, (float*)C, ldc, M, N, K, epi, stream)
                                   : launch_stream<NT, bf16>(X, ldx, W, ldw, (bf16*)C, ldc, M, N, K, epi, stream);
            if (st != kErrUnsupported) return st;
        }
    }
    if (out_f32) return launch_typed<NT, float>(X, ldx, W, ldw, (float*)C, ldc, M, N, K, epi, stream);
    return launch_typed<NT, bf16>(X, ldx, W, ldw, (bf16*)C, ldc, M, N, K, epi, stream);
}
}  // namespace

// 0, or 1 if a kernel of this file ever gave up waiting for its copies (reading
// it synchronises with the device).
GTG_API int gtg_gemm_bf16_skinny_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// Rows (tokens) this kernel takes.
GTG_API int gtg_gemm_bf16_skinny_max_rows() { return 64; }

// epilogue 0: C[M,N] = X W^T.  epilogue 1: W's rows come in blocks of 8 gate
// features followed by their 8 up features, and C[M,N/2] = silu(gate) * up.
GTG_API int gtg_gemm_bf16_skinny(const void* X, int ldx, const void* W, int ldw, void* C, int ldc,
                                 int out_f32, int M, int N, int K, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (epilogue != 0 && epilogue != 1) return kErrBadArgument;
    if (epilogue == 1 && N % 16 != 0) return kErrUnsupported;
    if (K <= 0 || ldx < K || ldw < K || ldc < (epilogue ? N / 2 : N)) return kErrBadArgument;
    if (M > 64) return kErrUnsupported;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    if ((N + 15) / 16 > 0x7fffffff / 16) return kErrUnsupported;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (M <= 8) return launch<1>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, epilogue, stream);
    if (M <= 16) return launch<2>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, epilogue, stream);
    if (M <= 32) return launch<4>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, epilogue, stream);
    return launch<8>(x, ldx, w, ldw, C, ldc, out_f32, M, N, K, epilogue, stream);
}

// ---- test hook --------------------------------------------------------------
// For the test that makes bounded waits run out: while `test_waits` is set, every
// launch of this library takes the kTest form of its kernel (see Waits above): no
// asynchronous copy is issued, so no barrier completes, and every wait gives up
// after a thousand polls.  Such a kernel returns without a result and the status
// word reads non-zero; nothing faults and nothing hangs.  The kernels as they
// normally run are not touched by this (the test form exists for bfloat16 results
// of up to 16 rows).  The call also clears the status word.
GTG_API int gtg_gemm_bf16_skinny_test_hooks(int test_waits) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    g_test_waits = test_waits != 0;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    return (int)e;
}

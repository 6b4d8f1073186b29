// bfloat16 product for decode batches of 17..64 tokens: C[M,N] = X[M,K] . W[N,K]^T.
//
// With this many tokens the work is still reading W once, but a CUDA-core or
// warp-level kernel would re-read X from L2 or shared memory several times per
// byte of W.  Here the roles of the operands are swapped on the tensor core:
// 128 rows of W are the M dimension of tcgen05.mma and the tokens (padded to 64)
// are its N dimension, so both operands go from shared memory to the tensor core
// once.  The accumulator [128 features x 64 tokens] lives in TMEM.
//
//   kernel 1  persistent, one CTA per SM.  A unit of work is (128-row tile of W,
//             slice of k); CTA c takes units c, c+G, c+2G ...  One thread keeps a
//             ring of eight 24 KB stages (a 128 x 64 block of W and the 64 x 64
//             block of X under it) full by TMA, across units; one thread issues
//             the MMAs as the stages land; four warps move finished accumulators
//             (two in TMEM, so a unit's epilogue runs under the next unit's MMAs)
//             to a float workspace [slice, token, feature].
//   kernel 2  adds the slices in order, applies the optional SwiGLU over
//             interleaved gate/up features, converts and stores C.
// The number of slices balances two costs: CTAs without work in the last round,
// and the workspace traffic, which grows with every slice.  Waits are bounded as
// in the other tcgen05 kernel; no cluster multicast is used.
#include "common.cuh"
#include <cuda.h>

namespace {
constexpr int BR = 128;                       // rows of W per CTA (MMA M)
constexpr int BT = 64;                        // tokens per CTA (MMA N)
constexpr int BK = 64;
constexpr int kStages = 8;                    // ring of k blocks
constexpr int kWBytes = BR * BK * 2, kXBytes = BT * BK * 2, kBlockBytes = kWBytes + kXBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 128;                // two accumulators of 64 columns
constexpr int kSmemBytes = kStages * kBlockBytes + 1024 + 256;
constexpr unsigned kSpinLimit = 1u << 22;

__device__ int g_status = 0;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                     "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(&g_status, 1);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major tile with 128-byte rows and 128-byte swizzle (see gemm_bf16_tcgen05.cu).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}

// part[slice][token][feature] (float), feature stride N.
__global__ void __launch_bounds__(kThreads)
swapab_partial_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      float* __restrict__ part, int M, int N, int K, int k_slice, int slices) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* aligned = smem_raw + (base - smem_addr(smem_raw));
    const uint32_t bars = base + kStages * kBlockBytes;      // full[kStages], empty[kStages], acc_full[2], acc_empty[2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    auto acc_full = [&](int a) { return bars + 8u * (2 * kStages + a); };
    auto acc_empty = [&](int a) { return bars + 8u * (2 * kStages + 2 + a); };
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(aligned + kStages * kBlockBytes + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kStages * kBlockBytes + 200);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_units = ((N + BR - 1) / BR) * slices;
    auto unit_k = [&](int unit, int* k_begin) {              // k blocks of the unit's slice
        *k_begin = (unit % slices) * k_slice;
        return (min(K, *k_begin + k_slice) - *k_begin + BK - 1) / BK;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_addr(tmem_holder)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // The first ring fill: the weights depend on no earlier kernel, so their
            // copies start before the wait; the activations follow it.
            uint32_t it = 0;
            bool waited = false, ok = true;
            int held[kStages][2];                            // (k, stage) of W copies whose X copy is still owed
            int n_held = 0;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                int k_begin;
                const int n_kb = unit_k(unit, &k_begin);
                const int n0 = (unit / slices) * BR;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!waited && it == kStages) {          // the ring is full of weights: now the activations
                        chain_wait();
                        for (int h = 0; h < n_held; ++h)
                            tma_load_2d(base + held[h][1] * kBlockBytes + kWBytes, &map_x, held[h][0], 0, full_bar(held[h][1]));
                        waited = true;
                    }
                    if (!mbar_wait(empty_bar(s), ((it / kStages) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), kBlockBytes);
                    tma_load_2d(base + s * kBlockBytes, &map_w, k_begin + kb * BK, n0, full_bar(s));
                    if (waited) {
                        tma_load_2d(base + s * kBlockBytes + kWBytes, &map_x, k_begin + kb * BK, 0, full_bar(s));
                    } else {
                        held[n_held][0] = k_begin + kb * BK;
                        held[n_held][1] = s;
                        ++n_held;
                    }
                }
            }
            if (!waited) {                                   // fewer blocks than stages in all
                chain_wait();
                for (int h = 0; h < n_held; ++h)
                    tma_load_2d(base + held[h][1] * kBlockBytes + kWBytes, &map_x, held[h][0], 0, full_bar(held[h][1]));
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BR, BT);
            uint32_t it = 0, done = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ++done) {
                int k_begin;
                const int n_kb = unit_k(unit, &k_begin);
                const int a = done & 1;
                if (!mbar_wait(acc_empty(a), ((done >> 1) & 1u) ^ 1u, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(full_bar(s), (it / kStages) & 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                    const uint64_t da = umma_desc(base + s * kBlockBytes);
                    const uint64_t db = umma_desc(base + s * kBlockBytes + kWBytes);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)
                        umma(tmem_base + 64 * a, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));               // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(acc_full(a));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: TMEM -> workspace
        chain_wait();                                       // the workspace may still be read by an earlier kernel
        uint32_t done = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++done) {
            const int a = done & 1;
            const bool ready = mbar_wait(acc_full(a), (done >> 1) & 1u, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
            const int feature = (unit / slices) * BR + warp * 32 + lane;
            float* dst = part + (size_t)(unit % slices) * M * N + feature;
#pragma unroll 1
            for (int c = 0; c < BT / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(tmem_base + 64 * a + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (feature < N) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int token = c * 32 + i;
                        if (token < M) dst[(size_t)token * N] = __uint_as_float(v[i]);   // a warp writes 32 consecutive features
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(a));
        }
    }
    chain_release();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
    }
}

// C[m][n] = sum over slices, in order; epi 1: SwiGLU over blocks of 8 gate + 8 up features.
template <typename OutT>
__global__ void swapab_reduce_kernel(const float* __restrict__ part, OutT* __restrict__ C, int ldc,
                                     int M, int N, int slices, int epi) {
    chain_wait();
    chain_release();
    const int n_out = epi ? N / 2 : N;
    const size_t total = (size_t)M * n_out;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(idx / n_out), j = (int)(idx - (size_t)m * n_out);
        if (!epi) {
            float s = 0.f;
            for (int sl = 0; sl < slices; ++sl) s += part[((size_t)sl * M + m) * N + j];
            C[(size_t)m * ldc + j] = from_f32<OutT>(s);
        } else {
            const int col = (j >> 3) * 16 + (j & 7);     // gate feature j; its up feature is 8 further
            float g = 0.f, u = 0.f;
            for (int sl = 0; sl < slices; ++sl) {
                const float* row = part + ((size_t)sl * M + m) * N;
                g += row[col];
                u += row[col + 8];
            }
            C[(size_t)m * ldc + j] = from_f32<OutT>(g / (1.0f + expf(-g)) * u);
        }
    }
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
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (!enc) return kErrUnsupported;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrBadArgument;
}

// Slices of k per row tile.  More slices fill the last round of the persistent
// grid better but add workspace traffic (every slice writes and re-reads M x 128
// floats per tile against 128 x k_slice weights): take the count with the least
// estimated time.
void plan(int M, int N, int K, int* slices, int* k_slice) {
    const int row_tiles = (N + BR - 1) / BR, k_blocks = (K + BK - 1) / BK, grid = 148;
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= k_blocks && s <= 64; ++s) {
        const int per = (k_blocks + s - 1) / s;                 // k blocks per slice
        const int real = (k_blocks + per - 1) / per;            // slices that exist with this size
        if (real != s) continue;
        const long long units = (long long)row_tiles * s;
        const long long rounds = (units + grid - 1) / grid;
        const double weights = (double)per * BK * 2 * BR, spill = 2.0 * M * 4 * BR;   // bytes per unit
        const double cost = (double)rounds * (weights + spill + 4096.0);              // + a fixed cost per unit
        if (cost < best_cost) { best_cost = cost; best = s; }
    }
    const int per = (k_blocks + best - 1) / best;
    *k_slice = per * BK;
    *slices = best;
}
}  // namespace

GTG_API int gtg_gemm_bf16_swapab_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// Floats of workspace a call needs.
GTG_API long long gtg_gemm_bf16_swapab_scratch_floats(int M, int N, int K) {
    int slices, k_slice;
    plan(M, N, K, &slices, &k_slice);
    return (long long)slices * M * N;
}

// M <= 64.  epilogue as in gtg_gemm_bf16_tcgen05.
GTG_API int gtg_gemm_bf16_swapab(const void* X, int ldx, const void* W, int ldw, void* C, int ldc,
                                 int out_f32, int M, int N, int K, int epilogue, float* scratch,
                                 cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > BT) return kErrUnsupported;
    if (epilogue != 0 && epilogue != 1) return kErrBadArgument;
    if (epilogue == 1 && N % 16 != 0) return kErrUnsupported;
    if (K <= 0 || ldx < K || ldw < K || ldc < (epilogue ? N / 2 : N) || scratch == nullptr) return kErrBadArgument;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    int slices, k_slice;
    plan(M, N, K, &slices, &k_slice);
    CUtensorMap map_w, map_x;
    int st = make_map(&map_w, W, N, K, ldw, BR);
    if (st != 0) return st;
    st = make_map(&map_x, X, M, K, ldx, BT);
    if (st != 0) return st;
    static bool configured = false;
    static int sms = 148;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(swapab_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        configured = true;
    }
    const long long units = (long long)((N + BR - 1) / BR) * slices;
    if (units > 0x7fffffff) return kErrUnsupported;
    const int grid = (int)(units < sms ? units : sms);
    st = launch_chained(swapab_partial_kernel, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream,
                        map_w, map_x, scratch, M, N, K, k_slice, slices);
    if (st != 0) return st;
    const int n_out = epilogue ? N / 2 : N;
    int blocks = (int)(((long long)M * n_out + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (out_f32)
        return launch_chained(swapab_reduce_kernel<float>, dim3(blocks), dim3(256), 0, stream,
                              (const float*)scratch, (float*)C, ldc, M, N, slices, epilogue);
    return launch_chained(swapab_reduce_kernel<bf16>, dim3(blocks), dim3(256), 0, stream,
                          (const float*)scratch, (bf16*)C, ldc, M, N, slices, epilogue);
}

// bfloat16 product for decode batches of 17..128 tokens: C[M,N] = X[M,K] . W[N,K]^T.
//
// With this many tokens the work is still reading W once, but a CUDA-core or
// warp-level kernel would re-read X from L2 or shared memory several times per
// byte of W.  Here the roles of the operands are swapped on the tensor core:
// 128 rows of W are the M dimension of tcgen05.mma and the tokens (padded to 32,
// 48, 64, 80 or 128) are its N dimension, so both operands go from shared memory
// to the tensor core once.  The accumulator [128 features x tokens] lives in TMEM.
//
// One CTA takes one (128-row tile of W, slice of k), two CTAs to an SM.  One
// thread keeps a ring of stages (a 128 x 64 block of W, 16 KB, and the block of X
// under it: five stages at up to 48 tokens, four at up to 80, three of 32 KB at
// 128) full by TMA -- the weights from before the wait on the kernel before, the
// activations after it -- one thread issues the MMAs as the
// stages land, and four warps move the finished accumulator to shared memory.
// The slices of a row tile are the CTAs of one thread-block cluster (up to
// eight): after a cluster barrier every CTA adds up, for its share of the
// tokens, the slices' partial sums in rank order through distributed shared
// memory, applies the optional SwiGLU over interleaved gate/up features,
// converts and stores C.  No workspace in global memory and no second kernel.
// The number of slices is what fills the SMs (two CTAs each) without cutting k
// below four blocks.  Waits are bounded as in the other tcgen05 kernel; no
// cluster multicast is used.
#include "common.cuh"
#include <cuda.h>

namespace {
constexpr int BR = 128;                       // rows of W per CTA (MMA M)
constexpr int BK = 64;
constexpr int kWBytes = BR * BK * 2;
constexpr int kThreads = 192;
constexpr int kCtasPerSm = 2;                 // what the ring's size lets an SM hold
constexpr int kMaxSlices = 8;                 // CTAs of a cluster (the portable limit)
// What depends on the tokens a CTA takes (BT, the MMA's N: 32, 48, 64, 80 or 128, the
// least that holds the step's rows): the stage (a 16 KB block of W and BT x 64 of X),
// as many stages as let two CTAs share an SM, the accumulator's TMEM columns.  The
// fewer tokens, the smaller X's share of a stage and the more stages there are.
template <int BT> struct Tile {
    static_assert(BT % 16 == 0 && BT >= 32 && BT <= 128, "the MMA's N");
    static constexpr int kStages = BT <= 48 ? 5 : BT <= 80 ? 4 : 3;   // ring of k blocks
    static constexpr int kXBytes = BT * BK * 2, kBlockBytes = kWBytes + kXBytes;
    static constexpr int kTmemCols = BT <= 32 ? 32 : BT <= 64 ? 64 : 128;   // one accumulator: 128 lanes x BT columns (a power of two is allocated)
    static constexpr int kPartFloats = BT * BR;                   // the accumulator as [token][feature], after the ring is done
    static constexpr int kSmemBytes = kStages * kBlockBytes + 1024 + 256;
    static_assert(kPartFloats * 4 <= kStages * kBlockBytes, "the partial sums reuse the ring");
    static_assert(2 * (kSmemBytes + 1024) <= 228 * 1024, "two CTAs share an SM");
    static_assert(kBlockBytes % 1024 == 0, "the swizzled tiles of every stage start on 1024 bytes");
    static_assert((2 * kStages + 1) * 8 <= 192, "the barriers lie below the TMEM holder");
};
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
template <bool kTest>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < Waits<kTest>::kLimit; ++i) {
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
template <bool kTest>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    if (Waits<kTest>::kSkipCopies) return;
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
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Four consecutive floats at `addr` of this CTA's shared memory, read from the CTA of rank `rank`.
__device__ __forceinline__ float4 remote_ld4(uint32_t addr, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra) : "memory");
    return v;
}

// grid.x = row tiles x slices, clusters of `slices` CTAs along x: CTA rank r of a
// cluster takes k blocks [r * kb_per, (r + 1) * kb_per) of its row tile.
template <typename OutT, int BT, bool kTest>
__global__ void __launch_bounds__(kThreads)
swapab_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
              OutT* __restrict__ C, int ldc, int M, int N, int K, int kb_per, int slices, int epi) {
    constexpr int kStages = Tile<BT>::kStages, kBlockBytes = Tile<BT>::kBlockBytes, kTmemCols = Tile<BT>::kTmemCols;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
    unsigned char* aligned = smem_raw + (base - smem_addr(smem_raw));
    const uint32_t bars = base + kStages * kBlockBytes;      // full[kStages], empty[kStages], acc_full
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    const uint32_t acc_full = bars + 8u * (2 * kStages);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(aligned + kStages * kBlockBytes + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + kStages * kBlockBytes + 200);
    float* part = reinterpret_cast<float*>(aligned);         // [token][feature], once the ring has been read
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = slices > 1 ? cluster_rank() : 0u;
    const int n0 = (blockIdx.x / slices) * BR;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_begin = (int)rank * kb_per;
    const int n_kb = max(0, min(kb_total, kb_begin + kb_per) - kb_begin);
    // CTAs of different row tiles walk the same k blocks of X: each starts at another
    // block, so that they do not all ask the L2 for the same lines at the same time
    const int kb_rot = n_kb > 0 ? (int)((blockIdx.x / slices) * 5u % (unsigned)n_kb) : 0;
    auto k_of = [&](int kb) { int j = kb + kb_rot; if (j >= n_kb) j -= n_kb; return (kb_begin + j) * BK; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(acc_full, 1);
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
    chain_release();      // the kernel after this one may set itself up; it waits for this one before it reads

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            // The first ring fill: the weights depend on no earlier kernel, so their
            // copies start before the wait; the activations follow it.
            const int first = min(n_kb, kStages);
            for (int kb = 0; kb < first; ++kb) {
                mbar_expect_tx(full_bar(kb), kBlockBytes);
                tma_load_2d<kTest>(base + kb * kBlockBytes, &map_w, k_of(kb), n0, full_bar(kb));
            }
            chain_wait();
            for (int kb = 0; kb < first; ++kb)
                tma_load_2d<kTest>(base + kb * kBlockBytes + kWBytes, &map_x, k_of(kb), 0, full_bar(kb));
            for (int kb = first; kb < n_kb; ++kb) {
                const int s = kb % kStages;
                if (!mbar_wait<kTest>(empty_bar(s), ((kb / kStages) & 1u) ^ 1u, abort_flag)) break;
                mbar_expect_tx(full_bar(s), kBlockBytes);
                tma_load_2d<kTest>(base + s * kBlockBytes, &map_w, k_of(kb), n0, full_bar(s));
                tma_load_2d<kTest>(base + s * kBlockBytes + kWBytes, &map_x, k_of(kb), 0, full_bar(s));
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BR, BT);
            bool ok = true;
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % kStages;
                if (!mbar_wait<kTest>(full_bar(s), (kb / kStages) & 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                const uint64_t da = umma_desc(base + s * kBlockBytes);
                const uint64_t db = umma_desc(base + s * kBlockBytes + kWBytes);
#pragma unroll
                for (int j = 0; j < BK / 16; ++j)
                    umma(tmem_base, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));                   // the stage is free once these MMAs have read it
            }
            if (ok && n_kb > 0) umma_commit(acc_full);       // arrives when every MMA above has completed
            else mbar_arrive(acc_full);                      // nothing to wait for (or given up): let the epilogue go on
        }
    } else {
        // ------------------------------------------------------------ accumulator -> shared memory, [token][feature]
        chain_wait();
        const bool ready = mbar_wait<kTest>(acc_full, 0u, abort_flag);
        const bool use = __all_sync(0xffffffffu, ready) && n_kb > 0 && !*abort_flag;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
        const int feature = warp * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BT / 16; ++c) {
            uint32_t v[16];
            if (use) {
                tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 16), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0u;      // a slice without k blocks adds nothing
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) part[(c * 16 + i) * BR + feature] = __uint_as_float(v[i]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    }
    // Every thread of every CTA of the cluster comes here, whatever its role did.
    __syncthreads();
    if (slices > 1) cluster_sync_all();                      // all slices' partial sums are in place

    if (warp < 4) {
        // this CTA's share of the tokens: the slices added in rank order, then the epilogue
        const int per = (BT + slices - 1) / slices;
        const int t_end = min(min(BT, M), (int)(rank + 1) * per);
        const uint32_t part_addr = smem_addr(part);
        const bool vec_ok = (ldc % 4 == 0) && (((uintptr_t)C) % 16 == 0);
        for (int t = (int)rank * per + warp; t < t_end; t += 4) {
            float4 acc;
            if (slices > 1) {
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int r = 0; r < slices; ++r) {
                    const float4 v = remote_ld4(part_addr + (uint32_t)(t * BR + lane * 4) * 4u, (uint32_t)r);
                    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                }
            } else {
                acc = *reinterpret_cast<const float4*>(part + t * BR + lane * 4);
            }
            if (!epi) {
                const int f = n0 + lane * 4;
                OutT* dst = C + (size_t)t * ldc + f;
                if (vec_ok && f + 3 < N) {
                    if constexpr (sizeof(OutT) == 4) {
                        *reinterpret_cast<float4*>(dst) = acc;
                    } else {
                        uint2 o;
                        o.x = pack_bf16x2(acc.x, acc.y);
                        o.y = pack_bf16x2(acc.z, acc.w);
                        *reinterpret_cast<uint2*>(dst) = o;
                    }
                } else {
                    const float a[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (f + i < N) dst[i] = from_f32<OutT>(a[i]);
                }
            } else {
                // features come in blocks of 8 gate + 8 up: lane l holds 4 of one half of block l / 4;
                // the matching half sits two lanes further (gate in lanes 4b, 4b+1; up in 4b+2, 4b+3)
                const float4 other = make_float4(__shfl_xor_sync(0xffffffffu, acc.x, 2), __shfl_xor_sync(0xffffffffu, acc.y, 2),
                                                 __shfl_xor_sync(0xffffffffu, acc.z, 2), __shfl_xor_sync(0xffffffffu, acc.w, 2));
                if ((lane & 2) == 0) {
                    const float g[4] = {acc.x, acc.y, acc.z, acc.w}, u[4] = {other.x, other.y, other.z, other.w};
                    const int j = (n0 >> 1) + (lane >> 2) * 8 + (lane & 1) * 4;     // first of this lane's four outputs
                    OutT* dst = C + (size_t)t * ldc + j;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (j + i < (N >> 1)) dst[i] = from_f32<OutT>(g[i] / (1.0f + expf(-g[i])) * u[i]);
                }
            }
        }
    }
    if (slices > 1) cluster_sync_all();                      // nobody leaves while its partial sums are being read
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
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

// Slices of k per row tile: as many as fill the device's CTA slots (two to an SM)
// without cutting k below four blocks a slice, at most eight (one cluster), and
// such that every slice has blocks.
void plan(int N, int K, int sms, int* slices, int* kb_per) {
    const int row_tiles = (N + BR - 1) / BR, k_blocks = (K + BK - 1) / BK;
    int s = (kCtasPerSm * sms) / row_tiles;
    if (s > kMaxSlices) s = kMaxSlices;
    if (s > k_blocks / 4) s = k_blocks / 4;
    if (s < 1) s = 1;
    while (s & (s - 1)) s &= s - 1;                           // a power of two: clusters of 3, 5, 6 or 7 CTAs pack the
                                                              // processor clusters unevenly and run in two waves
    int per = (k_blocks + s - 1) / s;
    s = (k_blocks + per - 1) / per;                           // slices that exist with this size
    *slices = s;
    *kb_per = per;
}

int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        else
            sms = 148;
    }
    return sms;
}

template <typename OutT, int BT, bool kTest>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, OutT* C, int ldc, int M, int N, int K,
           int kb_per, int slices, int epilogue, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(swapab_kernel<OutT, BT, kTest>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Tile<BT>::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long ctas = (long long)((N + BR - 1) / BR) * slices;
    if (ctas > 0x7fffffff) return kErrUnsupported;
    return launch_chained_cluster(swapab_kernel<OutT, BT, kTest>, dim3((unsigned)ctas), dim3(kThreads), slices,
                                  (size_t)Tile<BT>::kSmemBytes,
                                  stream, map_w, map_x, C, ldc, M, N, K, kb_per, slices, epilogue);
}
}  // namespace

GTG_API int gtg_gemm_bf16_swapab_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// Floats of workspace a call needs: none, the slices meet in shared memory.
GTG_API long long gtg_gemm_bf16_swapab_scratch_floats(int M, int N, int K) {
    (void)M; (void)N; (void)K;
    return 0;
}

// M <= 128.  epilogue as in gtg_gemm_bf16_tcgen05.  `scratch` is not used and may be null.
GTG_API int gtg_gemm_bf16_swapab(const void* X, int ldx, const void* W, int ldw, void* C, int ldc,
                                 int out_f32, int M, int N, int K, int epilogue, float* scratch,
                                 cudaStream_t stream) {
    (void)scratch;
    if (M <= 0 || N <= 0) return 0;
    if (M > 128) return kErrUnsupported;
    if (epilogue != 0 && epilogue != 1) return kErrBadArgument;
    if (epilogue == 1 && N % 16 != 0) return kErrUnsupported;
    if (K <= 0 || ldx < K || ldw < K || ldc < (epilogue ? N / 2 : N)) return kErrBadArgument;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    int slices, kb_per;
    plan(N, K, device_sms(), &slices, &kb_per);
    // tokens a CTA takes, the MMA's N: the least of these that holds the rows
    int bt = M <= 32 ? 32 : M <= 48 ? 48 : M <= 64 ? 64 : M <= 80 ? 80 : 128;
    if (g_test_waits) bt = M <= 64 ? 64 : 128;              // the give-up test's form exists for 64 tokens
    CUtensorMap map_w, map_x;
    int st = make_map(&map_w, W, N, K, ldw, BR);
    if (st != 0) return st;
    st = make_map(&map_x, X, M, K, ldx, bt);
    if (st != 0) return st;
#define GTG_ARGS(T) map_w, map_x, (T*)C, ldc, M, N, K, kb_per, slices, epilogue, stream
    if (g_test_waits) {                                      // the give-up test: up to 64 rows
        if (bt != 64) return kErrUnsupported;
        return out_f32 ? launch<float, 64, true>(GTG_ARGS(float)) : launch<bf16, 64, true>(GTG_ARGS(bf16));
    }
    if (bt == 32) return out_f32 ? launch<float, 32, false>(GTG_ARGS(float)) : launch<bf16, 32, false>(GTG_ARGS(bf16));
    if (bt == 48) return out_f32 ? launch<float, 48, false>(GTG_ARGS(float)) : launch<bf16, 48, false>(GTG_ARGS(bf16));
    if (bt == 64) return out_f32 ? launch<float, 64, false>(GTG_ARGS(float)) : launch<bf16, 64, false>(GTG_ARGS(bf16));
    if (bt == 80) return out_f32 ? launch<float, 80, false>(GTG_ARGS(float)) : launch<bf16, 80, false>(GTG_ARGS(bf16));
    return out_f32 ? launch<float, 128, false>(GTG_ARGS(float)) : launch<bf16, 128, false>(GTG_ARGS(bf16));
#undef GTG_ARGS
}

// ---- test hook --------------------------------------------------------------
// For the test that makes bounded waits run out: while `test_waits` is set, every
// launch of this library takes the kTest form of its kernel (see Waits above): no
// asynchronous copy is issued, so no barrier completes, and every wait gives up
// after a thousand polls.  Such a kernel returns without a result and the status
// word reads non-zero; nothing faults and nothing hangs.  The kernels as they
// normally run are not touched by this.  The call also clears the status word.
GTG_API int gtg_gemm_bf16_swapab_test_hooks(int test_waits) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    g_test_waits = test_waits != 0;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    return (int)e;
}

// bfloat16 matrix product on the fifth-generation tensor cores:
//   C[M,N] = A[M,K] . W[N,K]^T,  float accumulation in tensor memory (TMEM),
// output bfloat16 or float.  Both operands are K-major, W as in the checkpoint.
//
// Persistent CTAs, one per SM, each walking 128 x 256 tiles of C (tile index
// = m + n * tiles_m, so that the CTAs running at one time share the rows of A
// and read each tile of W once).  Roles by warp:
//   warps 0-3  epilogue: tcgen05.ld the accumulator (warp w owns TMEM lanes
//              32w..32w+31 = rows of the tile), optional SwiGLU, convert, store
//   warp 4     producer: one thread issues the TMA loads (cp.async.bulk.tensor,
//              128-byte swizzle) of the A tile (128 x 64) and the W tile
//              (256 x 64) of each k block into a four-stage ring that runs on
//              across tiles
//   warp 5     allocates TMEM; one thread issues tcgen05.mma (128 x 256 x 16,
//              four per k block) and releases ring stages with tcgen05.commit
// TMEM holds two accumulators (2 x 256 columns): while the epilogue drains one,
// the MMAs of the next tile fill the other.
// Rows and columns beyond M, N and the tail of K are zero-filled by TMA and
// dropped at the store, so any M and N work; K must be a multiple of 8 (the
// 16-byte row pitch TMA needs).
//
// Every wait on an mbarrier is bounded.  A wait that gives up sets a flag in
// shared memory that makes all roles fall through to the common exit (where TMEM
// is released) and records it in a status word the host can read
// (gtg_gemm_bf16_tcgen05_status).  No cluster multicast is used anywhere.
#include "common.cuh"
#include <cuda.h>

namespace {
constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int kThreads = 192;
constexpr int kABytes = BM * BK * 2, kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 512;                     // two accumulators of BN columns
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

constexpr int kStoreBytes = 32 * 128;              // one staged box: 32 rows x 64 bfloat16
constexpr int kSmemBytes = STAGES * kStageBytes + 1024 /* barriers */ + 4 * 2 * kStoreBytes /* staging */ +
                           1024 /* alignment slack */;

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
// Polls until the phase with `parity` completes, the abort flag is raised, or the limit is hit.
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
// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64
// bfloat16), 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);             // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
    d |= (uint64_t)1 << 46;                              // version
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}
// Instruction descriptor of kind::f16: float accumulator, bfloat16 A and B, both K-major.
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

// n_valid values (float bits in v) to dst; 16-byte stores when the row allows.
template <typename OutT, int n_full>
__device__ __forceinline__ void store_values(OutT* dst, const uint32_t* v, int n_valid, bool vec_ok) {
    if (vec_ok && n_valid == n_full) {
        if constexpr (sizeof(OutT) == 2) {
#pragma unroll
            for (int i = 0; i < n_full / 8; ++i) {
                uint32_t p[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]),
                                                             __uint_as_float(v[8 * i + 2 * j + 1]));
                    p[j] = *reinterpret_cast<uint32_t*>(&h);
                }
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[0], p[1], p[2], p[3]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < n_full / 4; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
    } else {
        for (int i = 0; i < n_valid; ++i) dst[i] = from_f32<OutT>(__uint_as_float(v[i]));
    }
}

// For epilogue 2 (the fused query/key/value projection of heads of 64 channels):
// where a token's rotation table, cache page and place in the page are found.
struct RopeKV {
    const float2* cos_sin;       // [M][32] (cos, sin) of the token's position
    const int* token_seq;        // [M] sequence of the step each token belongs to
    const int* slots;            // [sequences] cache slot
    const int* positions;        // [M]
    const int* block_table;
    int table_stride;
    bf16* kc;                    // the cache entry's keys and values
    bf16* vc;
    long long page_stride;
    int n_heads, n_kv;
};

template <typename OutT, bool kTest>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c, int use_store_map,
                    OutT* __restrict__ C, int ldc, int M, int N, int K, int epi, RopeKV rope) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;        // tiles need 1024-byte alignment
    unsigned char* aligned = smem_raw + (base - smem_addr(smem_raw));
    const uint32_t bars = base + STAGES * kStageBytes;   // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(aligned + STAGES * kStageBytes + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(aligned + STAGES * kStageBytes + 136);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;
    const int n_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full_bar(a), 1); mbar_init(acc_empty_bar(a), 4); }
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
    // Barriers and tensor memory are set up; from here on the kernel reads and
    // writes what the kernel before it may still be using.
    chain_wait();
    chain_release();

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t it = 0;                                   // k blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    ok = mbar_wait<kTest>(empty_bar(s), (round & 1u) ^ 1u, abort_flag);   // passes at once in round 0
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), kStageBytes);
                    tma_load_2d<kTest>(base + s * kStageBytes, &map_a, kb * BK, m0, full_bar(s));
                    tma_load_2d<kTest>(base + s * kStageBytes + kABytes, &map_w, kb * BK, n0, full_bar(s));
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(BM, BN);
            uint32_t it = 0;
            bool ok = true;
            int t = 0;                                         // tiles done by this CTA
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
                const int acc = t & 1;
                ok = mbar_wait<kTest>(acc_empty_bar(acc), (((uint32_t)t >> 1) & 1u) ^ 1u, abort_flag);   // epilogue drained it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                const uint32_t tmem_acc = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    ok = mbar_wait<kTest>(full_bar(s), round & 1u, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                    const uint64_t da = umma_desc(base + s * kStageBytes);
                    const uint64_t db = umma_desc(base + s * kStageBytes + kABytes);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)           // 32 bytes (16 values of k) further per step
                        umma(tmem_acc, da + 2 * j, db + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    umma_commit(empty_bar(s));                  // the stage is free once these MMAs have read it
                }
                umma_commit(acc_full_bar(acc));                 // this accumulator is complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const bool vec_ok = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        // bfloat16 rows that TMA can address: the warp stages 32 rows x 64 columns in
        // shared memory (128-byte rows, swizzled like the tensor map) and one lane
        // stores the box; the store clips rows and columns beyond M and the output
        // width.  Otherwise every lane stores its own row directly.
        const bool staged = use_store_map && sizeof(OutT) == 2;
        unsigned char* stage_base = aligned + STAGES * kStageBytes + 1024 + warp * (2 * kStoreBytes);
        uint32_t groups = 0;                               // 64-column boxes stored so far by this warp
        int t = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            const int acc = t & 1;
            if (!mbar_wait<kTest>(acc_full_bar(acc), ((uint32_t)t >> 1) & 1u, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
            const int row = m0 + warp * 32 + lane;
            const uint32_t tmem_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * BN);
            if (epi == 2) {
                // Query/key/value heads of 64 channels: a box of 64 columns is one head, its two
                // chunks hold the rotation's pairs (d, d + 32).  Query heads are rotated and stored
                // like any output; key heads are rotated and written into the token's cache page,
                // value heads are copied there (the projection's key and value columns are not stored).
                const bool live = row < M;
                size_t cache_at = 0;                       // of (key/value head 0, this token, channel 0)
                if (live) {
                    const int pos = rope.positions[row];
                    const int page = rope.block_table[(size_t)rope.slots[rope.token_seq[row]] * rope.table_stride + pos / kPageTokens];
                    cache_at = (size_t)page * rope.page_stride + (size_t)(pos % kPageTokens) * 64;
                }
                const float4* cs = reinterpret_cast<const float4*>(rope.cos_sin + (size_t)(live ? row : 0) * 32);
#pragma unroll 1
                for (int c0 = 0; c0 < BN / 32; c0 += 2) {
                    const int col = n0 + c0 * 32;
                    if (col >= N) break;
                    const int head = col >> 6;
                    uint32_t v0[32], v1[32];
                    tmem_ld32(tmem_row + (uint32_t)(c0 * 32), v0);
                    tmem_ld32(tmem_row + (uint32_t)((c0 + 1) * 32), v1);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (head < rope.n_heads + rope.n_kv) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float4 t = cs[i >> 1];   // (cos, sin) of channels i and i + 1
                            const float a0 = __uint_as_float(v0[i]), b0 = __uint_as_float(v1[i]);
                            const float a1 = __uint_as_float(v0[i + 1]), b1 = __uint_as_float(v1[i + 1]);
                            v0[i] = __float_as_uint(a0 * t.x - b0 * t.y);
                            v1[i] = __float_as_uint(a0 * t.y + b0 * t.x);
                            v0[i + 1] = __float_as_uint(a1 * t.z - b1 * t.w);
                            v1[i + 1] = __float_as_uint(a1 * t.w + b1 * t.z);
                        }
                    }
                    // 64 values -> eight 16-byte pieces
                    uint4 pieces[8];
#pragma unroll
                    for (int piece = 0; piece < 4; ++piece) {
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v0[8 * piece + 2 * q]),
                                                                      __uint_as_float(v0[8 * piece + 2 * q + 1]));
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v1[8 * piece + 2 * q]),
                                                                      __uint_as_float(v1[8 * piece + 2 * q + 1]));
                            lo[q] = *reinterpret_cast<uint32_t*>(&h0);
                            hi[q] = *reinterpret_cast<uint32_t*>(&h1);
                        }
                        pieces[piece] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        pieces[piece + 4] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    }
                    if (head < rope.n_heads) {
                        unsigned char* buf = stage_base + (groups & 1u) * kStoreBytes;
                        if (groups >= 2) {                 // the box stored from this buffer two rounds ago has been read
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                            __syncwarp();
                        }
#pragma unroll
                        for (int piece = 0; piece < 8; ++piece)
                            *reinterpret_cast<uint4*>(buf + lane * 128 + ((piece ^ (lane & 7)) << 4)) = pieces[piece];
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> TMA reads
                        __syncwarp();
                        if (lane == 0) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];\n"
                                         ::"l"(&map_c), "r"(smem_addr(buf)), "r"(col), "r"(m0 + warp * 32) : "memory");
                            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                        }
                        ++groups;
                    } else if (live) {
                        const bool is_key = head < rope.n_heads + rope.n_kv;
                        const int kvh = head - rope.n_heads - (is_key ? 0 : rope.n_kv);
                        uint4* dst = reinterpret_cast<uint4*>((is_key ? rope.kc : rope.vc) + cache_at +
                                                              (size_t)kvh * kPageTokens * 64);
#pragma unroll
                        for (int piece = 0; piece < 8; ++piece) dst[piece] = pieces[piece];
                    }
                }
            } else if (epi == 3) {
                // C is a float residual stream and map_c describes it in boxes of 32 columns x 32
                // rows: every chunk of the accumulator, rounded to bfloat16 as a stored update
                // would be, is staged as 32 rows of 128 bytes and ADDED to the residual by the
                // copy engine (one tensor reduction per box; each element is added once).
#pragma unroll 1
                for (int c0 = 0; c0 < BN / 32; ++c0, ++groups) {
                    if (n0 + c0 * 32 >= N) break;
                    unsigned char* buf = stage_base + (groups & 1u) * kStoreBytes;
                    if (groups >= 2) {                     // the box sent from this buffer two rounds ago has been read
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                        __syncwarp();
                    }
                    uint32_t v[32];
                    tmem_ld32(tmem_row + (uint32_t)(c0 * 32), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int piece = 0; piece < 8; ++piece) {
                        float f[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            f[q] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[4 * piece + q])));
                        *reinterpret_cast<float4*>(buf + lane * 128 + ((piece ^ (lane & 7)) << 4)) =
                            make_float4(f[0], f[1], f[2], f[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> TMA reads
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];\n"
                                     ::"l"(&map_c), "r"(smem_addr(buf)), "r"(n0 + c0 * 32), "r"(m0 + warp * 32) : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                }
            } else if (staged) {
                const int per_box = epi ? 4 : 2;           // accumulator chunks of 32 columns per 64 output columns
#pragma unroll 1
                for (int c0 = 0; c0 < BN / 32; c0 += per_box, ++groups) {
                    unsigned char* buf = stage_base + (groups & 1u) * kStoreBytes;
                    if (groups >= 2) {                     // the box stored from this buffer two rounds ago has been read
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
                        __syncwarp();
                    }
                    for (int cc = 0; cc < per_box; ++cc) {
                        uint32_t v[32];
                        tmem_ld32(tmem_row + (uint32_t)((c0 + cc) * 32), v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                        if (epi == 0) {
                            // 32 columns = four 16-byte pieces, at pieces 4*cc .. 4*cc+3 of the row
#pragma unroll
                            for (int piece = 0; piece < 4; ++piece) {
                                uint32_t p[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * piece + 2 * q]),
                                                                             __uint_as_float(v[8 * piece + 2 * q + 1]));
                                    p[q] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                const int chunk = 4 * cc + piece;
                                *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                                    make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        } else {
                            // SwiGLU: two blocks of 8 gate + 8 up features -> 16 outputs = two pieces
#pragma unroll
                            for (int blk = 0; blk < 2; ++blk) {
                                uint32_t p[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const float g0 = __uint_as_float(v[16 * blk + 2 * q]), u0 = __uint_as_float(v[16 * blk + 8 + 2 * q]);
                                    const float g1 = __uint_as_float(v[16 * blk + 2 * q + 1]), u1 = __uint_as_float(v[16 * blk + 9 + 2 * q]);
                                    __nv_bfloat162 h = __floats2bfloat162_rn(g0 / (1.0f + __expf(-g0)) * u0,
                                                                             g1 / (1.0f + __expf(-g1)) * u1);
                                    p[q] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                const int chunk = 2 * cc + blk;
                                *reinterpret_cast<uint4*>(buf + lane * 128 + ((chunk ^ (lane & 7)) << 4)) =
                                    make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes -> TMA reads
                    __syncwarp();
                    if (lane == 0) {
                        const int out_col = epi ? ((n0 + c0 * 32) >> 1) : (n0 + c0 * 32);
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];\n"
                                     ::"l"(&map_c), "r"(smem_addr(buf)), "r"(out_col), "r"(m0 + warp * 32) : "memory");
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld32(tmem_row + (uint32_t)(c * 32), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    const int col = n0 + c * 32;
                    if (row >= M || col >= N) continue;
                    if (epi == 0) {
                        store_values<OutT, 32>(C + (size_t)row * ldc + col, v, min(32, N - col), vec_ok);
                    } else {
                        // SwiGLU: the 32 columns are two blocks of 8 gate features followed by
                        // their 8 up features; 16 outputs land at column col/2
                        uint32_t o[16];
#pragma unroll
                        for (int blk = 0; blk < 2; ++blk)
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float g = __uint_as_float(v[16 * blk + q]), u = __uint_as_float(v[16 * blk + 8 + q]);
                                o[8 * blk + q] = __float_as_uint(g / (1.0f + __expf(-g)) * u);
                            }
                        store_values<OutT, 16>(C + (size_t)row * ldc + (col >> 1), o, min(16, (N - col) / 2), vec_ok);
                    }
                }
            }
            // all of this warp's reads of the accumulator are done: hand it back
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
        }
        if ((staged || epi == 3) && lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // stores have landed
    }
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

// A [rows, K] bfloat16 matrix with `ld` elements between rows, read in boxes of 64 x box_rows.
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
}  // namespace

// 0, or 1 if a kernel of this file ever gave up a bounded wait (reading it
// synchronises with the device).
GTG_API int gtg_gemm_bf16_tcgen05_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

namespace {
// epilogue 0: C[M,N] = A W^T.  1: SwiGLU over interleaved rows.  2: rotation and cache store (rope).
int run(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int out_f32, int M, int N, int K,
        int epilogue, const RopeKV& rope, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (epilogue < 0 || epilogue > 3) return kErrBadArgument;
    if (epilogue == 1 && N % 16 != 0) return kErrUnsupported;
    if (epilogue == 3 && (!out_f32 || ldc % 4 || ((uintptr_t)C % 16))) return kErrUnsupported;
    if (K <= 0 || lda < K || ldw < K || ldc < (epilogue == 1 ? N / 2 : N)) return kErrBadArgument;
    if (K % 8 || lda % 8 || ldw % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return kErrUnsupported;
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    if (tiles > 0x7fffffffLL) return kErrUnsupported;
    CUtensorMap map_a, map_w;
    int st = make_map(&map_a, A, M, K, lda, BM);
    if (st != 0) return st;
    st = make_map(&map_w, W, N, K, ldw, BN);
    if (st != 0) return st;
    // the store map: C as [M, output width] bfloat16 in boxes of 64 x 32 (when its rows allow it)
    const int n_out = epilogue == 1 ? N / 2 : N;
    CUtensorMap map_c = map_a;
    int use_store_map = 0;
    if (!out_f32 && ldc % 8 == 0 && ((uintptr_t)C % 16) == 0) {
        if (make_map(&map_c, C, M, n_out, ldc, 32) == 0) use_store_map = 1;
    }
    if (epilogue == 2 && !use_store_map) return kErrUnsupported;
    if (epilogue == 3) {
        // the residual stream as [M, N] float in boxes of 32 x 32 for the tensor reduction
        EncodeTiled enc = encode_fn();
        if (!enc) return kErrUnsupported;
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
        const cuuint32_t box[2] = {32u, 32u};
        const cuuint32_t elem[2] = {1, 1};
        if (enc(&map_c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, C, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return kErrUnsupported;
    }
    static bool configured = false;
    static int sms = 148;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gemm_tcgen05_kernel<bf16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gemm_tcgen05_kernel<bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(gemm_tcgen05_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            sms = n;
        configured = true;
    }
    const int grid = (int)(tiles < sms ? tiles : sms);
    if (g_test_waits) {
        if (out_f32)
            return launch_chained(gemm_tcgen05_kernel<float, true>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream,
                                  map_a, map_w, map_c, use_store_map, (float*)C, ldc, M, N, K, epilogue, rope);
        return launch_chained(gemm_tcgen05_kernel<bf16, true>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream,
                              map_a, map_w, map_c, use_store_map, (bf16*)C, ldc, M, N, K, epilogue, rope);
    }
    if (out_f32)
        return launch_chained(gemm_tcgen05_kernel<float, false>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream,
                              map_a, map_w, map_c, use_store_map, (float*)C, ldc, M, N, K, epilogue, rope);
    return launch_chained(gemm_tcgen05_kernel<bf16, false>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, stream,
                          map_a, map_w, map_c, use_store_map, (bf16*)C, ldc, M, N, K, epilogue, rope);
}
}  // namespace

// epilogue 0: C[M,N] = A W^T.  epilogue 1: W's rows come in blocks of 8 gate
// features followed by their 8 up features, and C[M,N/2] = silu(gate) * up.
GTG_API int gtg_gemm_bf16_tcgen05(const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                                  int out_f32, int M, int N, int K, int epilogue, cudaStream_t stream) {
    if (epilogue != 0 && epilogue != 1) return kErrBadArgument;
    return run(A, lda, W, ldw, C, ldc, out_f32, M, N, K, epilogue, RopeKV{}, stream);
}

// residual[M,N] (float, row pitch ldr) += bfloat16(A W^T): the update, rounded as a
// stored one would be, is added to the residual stream by tensor reductions in the
// epilogue.  Each element is added exactly once, so the result does not depend on
// timing.
GTG_API int gtg_gemm_bf16_tcgen05_add(const void* A, int lda, const void* W, int ldw, float* residual, int ldr,
                                      int M, int N, int K, cudaStream_t stream) {
    if (residual == nullptr) return kErrBadArgument;
    return run(A, lda, W, ldw, residual, ldr, 1, M, N, K, 3, RopeKV{}, stream);
}

// The query/key/value projection of heads of 64 channels with what follows it
// fused into the epilogue: W = [Wq; Wk; Wv] with (n_heads + 2 n_kv) * 64 rows;
// the query columns of C receive the rotated queries; rotated keys and the
// values go straight into the cache entry (kc, vc, page_stride, block_table) at
// each token's (slot, position); C's key and value columns are left untouched.
// cos_sin: float [M][32][2].
GTG_API int gtg_gemm_bf16_tcgen05_qkv_rope(const void* A, int lda, const void* W, int ldw, void* C, int ldc,
                                           int M, int K, const void* cos_sin, const int* token_seq,
                                           const int* slots, const int* positions, const int* block_table,
                                           int table_stride, void* kc, void* vc, long long page_stride,
                                           int n_heads, int n_kv, cudaStream_t stream) {
    if (n_heads <= 0 || n_kv <= 0 || cos_sin == nullptr || kc == nullptr || vc == nullptr) return kErrBadArgument;
    if (((uintptr_t)cos_sin % 16) || ((uintptr_t)kc % 16) || ((uintptr_t)vc % 16) || page_stride % 8) return kErrUnsupported;
    RopeKV rope{(const float2*)cos_sin, token_seq, slots, positions, block_table, table_stride,
                (bf16*)kc, (bf16*)vc, page_stride, n_heads, n_kv};
    return run(A, lda, W, ldw, C, ldc, 0, M, (n_heads + 2 * n_kv) * 64, K, 2, rope, stream);
}

// ---- test hook --------------------------------------------------------------
// For the test that makes bounded waits run out: while `test_waits` is set, every
// launch of this library takes the kTest form of its kernel (see Waits above): no
// asynchronous copy is issued, so no barrier completes, and every wait gives up
// after a thousand polls.  Such a kernel returns without a result and the status
// word reads non-zero; nothing faults and nothing hangs.  The kernels as they
// normally run are not touched by this.  The call also clears the status word.
GTG_API int gtg_gemm_bf16_tcgen05_test_hooks(int test_waits) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    g_test_waits = test_waits != 0;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    return (int)e;
}

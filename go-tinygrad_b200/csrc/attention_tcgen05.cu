// Causal grouped-query prefill attention on the fifth-generation tensor cores,
// for heads of 64 or 128 channels, over the paged cache.
//
// One CTA per (128-query tile, query head, sequence).  Per step of BK keys (two
// cache pages = 128 keys for heads of 64 channels, one page for heads of 128):
//   S  = Q K^T      tcgen05.mma 128 x BK x head size: Q and the key pages in shared
//                   memory (TMA, 128-byte swizzle, both K-major, 64 channels per
//                   swizzled block), S in TMEM
//   P  = softmax    four warps, one thread per query row: tcgen05.ld its BK scores
//                   into registers and hand the TMEM tile back at once (the next
//                   step's S runs under this step's softmax); mask (diagonal and
//                   window-edge steps only), running max and sum in float; the row
//                   of P goes back to TMEM as packed bfloat16 (tcgen05.st)
//   O += P V        tcgen05.mma 128 x head size x BK with A = P read from TMEM and
//                   the value pages as the MN-major B operand -- a page's
//                   [key][channel] rows are that layout as they lie in the cache --
//                   accumulating in TMEM over all steps
// Neither P nor O passes through shared memory, whose bandwidth is what limits
// small tiles on this machine.  The running maximum m of a row is only raised
// when the step's maximum exceeds it by more than 2^8; until then P = exp2(s - m)
// is taken against the older m (at most 256, exact in float and as good as any
// other scale in bfloat16) and the sum uses the same m, so the quotient O / l is
// unchanged.  Raising m multiplies the row of O in TMEM by exp2(m_old - m_new)
// (tcgen05.ld / st by the row's thread, after the previous product has completed);
// it happens in the first steps and rarely later.  Roles: warps 0-3 softmax and
// output, warp 4 issues the TMA loads (a ring of key + value pages), warp 5
// allocates TMEM and issues the MMAs.  Two CTAs share an SM (256 TMEM columns
// each).  Every mbarrier wait is bounded (status word as in the products).
#include "common.cuh"
#include <cuda.h>
#include <math.h>

namespace {
constexpr int BQ = 128;                 // query rows per CTA
constexpr int kThreads = 192;
constexpr int kBlockBytes = kPageTokens * 64 * 2;   // 64 tokens x 64 channels: one swizzled block of a page
constexpr int kTmemCols = 256;
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

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRaiseBy = 8.0f;        // the running maximum follows only jumps above 2^8

// Sizes that follow from the head size.
template <int HD> struct Shape {
    static constexpr int BK = HD == 64 ? 128 : 64;             // keys per step
    static constexpr int kPages = BK / kPageTokens;            // cache pages per step
    static constexpr int kHalves = HD / 64;                    // 64-channel blocks per row
    static constexpr int kStages = HD == 64 ? 3 : 2;           // steps of keys and values in flight
    static constexpr int kQBytes = BQ * HD * 2;
    static constexpr int kTileBytes = BK * HD * 2;             // the keys (or the values) of a step
    static constexpr int kStageBytes = 2 * kTileBytes;
    static constexpr int kOffKV = kQBytes;
    static constexpr int kOffBar = kOffKV + kStages * kStageBytes;
    static constexpr int kSmemBytes = kOffBar + 256;
    // TMEM columns: S (BK floats), O (HD floats), P (BK bfloat16 as pairs)
    static constexpr int kColO = BK, kColP = BK + HD;
    static_assert(BK + HD + BK / 2 <= kTmemCols, "tensor memory");
};

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
// Operand descriptor for blocks of 128-byte rows with 128-byte swizzle whose 8-row
// groups are 1024 bytes apart.  Read K-major (rows = M/N index, the 64 values of a
// row = k) or MN-major (rows = k index, the 64 values of a row = M/N index): which
// one is said by the instruction descriptor, the bytes are laid out the same.
// `mn_block_bytes`: for an MN-major operand wider than 64, the distance between
// its 64-wide blocks.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t mn_block_bytes = 16) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16, float accumulator, bfloat16 operands; A K-major; B K-major or MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[shared] B[shared]
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] B[shared]
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
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
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(addr),
                   "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_st8(uint32_t addr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// The same, kept in program order among its like (volatile), so that a batch of
// them stays a batch in the machine code.
__device__ __forceinline__ float exp2_in_order(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// map_q: the step's [tokens, row width] activations, boxes of 64 channels x 128 rows.
// map_kv: one cache entry as rows of HD channels, row = ((page*2 + k|v)*n_kv + head)*64 + token;
//         boxes of 64 channels x 64 rows.
// grid: (query heads, sequences, query tiles), the longest tiles first.
// A stage of the ring: the step's keys, then its values, each as HD/64 blocks of
// [BK tokens][64 channels] (a block holds the step's pages one after the other).
template <int HD, bool kTest>
__global__ void __launch_bounds__(kThreads, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            bf16* __restrict__ out, int ldo,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                            const int* __restrict__ start_pos,
                            int n_heads, int n_kv, float scale, int window) {
    using S = Shape<HD>;
    constexpr int BK = S::BK;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int h = blockIdx.x, b = blockIdx.y;
    const int tile = gridDim.z - 1 - blockIdx.z;
    const int q_begin = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_begin;
    if (tile * BQ >= q_len) return;                              // before any barrier or TMEM use
    const uint32_t base = smem_addr(smem);
    if (base & 1023u) {                                          // the swizzled tiles need this alignment
        if (threadIdx.x == 0) atomicExch(&g_status, 2);
        return;
    }
    const uint32_t bars = base + S::kOffBar;
    const uint32_t q_full = bars, s_full = bars + 8, s_free = bars + 16, p_full = bars + 24, pv_done = bars + 32;
    auto kv_full = [&](int s) { return bars + 40u + 8u * s; };
    auto kv_empty = [&](int s) { return bars + 40u + 8u * S::kStages + 8u * s; };
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + S::kOffBar + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::kOffBar + 136);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int start = start_pos[b];
    const int kvh = h / (n_heads / n_kv);
    const int* table = block_table + (size_t)slots[b] * table_stride;
    const int rows_here = min(BQ, q_len - tile * BQ);
    const int k_max = start + tile * BQ + rows_here - 1;         // last key any row of the tile sees
    const int k_min = window > 0 ? max(0, start + tile * BQ - window + 1) : 0;
    const int j_lo = k_min / kPageTokens, j_hi = k_max / kPageTokens;
    const int n_steps = (j_hi - j_lo + S::kPages) / S::kPages;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(s_full, 1);
        mbar_init(s_free, 4);                                    // one arrival per softmax warp
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
        for (int s = 0; s < S::kStages; ++s) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
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
    const uint32_t tmem_s = *tmem_holder, tmem_o = tmem_s + S::kColO, tmem_p = tmem_s + S::kColP;
    chain_wait();                                                // queries, keys and values come from the kernel before
    chain_release();

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, S::kQBytes);
            for (int hh = 0; hh < S::kHalves; ++hh)
                tma_load_2d<kTest>(base + hh * (BQ * 128), &map_q, h * HD + 64 * hh, q_begin + tile * BQ, q_full);
            for (int i = 0; i < n_steps; ++i) {
                const int s = i % S::kStages;
                if (!mbar_wait<kTest>(kv_empty(s), (((uint32_t)i / S::kStages) & 1u) ^ 1u, abort_flag)) break;
                const uint32_t dst = base + S::kOffKV + s * S::kStageBytes;
                mbar_expect_tx(kv_full(s), S::kStageBytes);
                for (int pg = 0; pg < S::kPages; ++pg) {
                    // a page beyond the last one is the step's first page again: finite values under keys that no row sees
                    const int j = j_lo + S::kPages * i + pg;
                    const int page = table[j <= j_hi ? j : j_lo + S::kPages * i];
                    for (int kv = 0; kv < 2; ++kv) {
                        const int row = ((page * 2 + kv) * n_kv + kvh) * kPageTokens;
                        for (int hh = 0; hh < S::kHalves; ++hh)
                            tma_load_2d<kTest>(dst + kv * S::kTileBytes + (hh * S::kPages + pg) * kBlockBytes, &map_kv,
                                        64 * hh, row, kv_full(s));
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(BQ, BK, 0);               // S[128 x BK keys], key pages K-major
            const uint32_t idesc_pv = umma_idesc(BQ, HD, 1);              // O[128 x HD channels], value pages MN-major
            bool ok = mbar_wait<kTest>(q_full, 0, abort_flag);
            auto issue_s = [&](int i) {
                const int s = i % S::kStages;
                if (!mbar_wait<kTest>(kv_full(s), ((uint32_t)i / S::kStages) & 1u, abort_flag)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                const uint32_t kbase = base + S::kOffKV + s * S::kStageBytes;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {                     // 16 channels per step, 64 per swizzled block
                    const uint64_t dq = umma_desc(base + (kk / 4) * (BQ * 128)) + 2 * (kk % 4);
                    const uint64_t dk = umma_desc(kbase + (kk / 4) * (BK * 128)) + 2 * (kk % 4);
                    umma_ss(tmem_s, dq, dk, idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(s_full);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int i = 0; i < n_steps && ok; ++i) {
                if (i + 1 < n_steps) {                                     // S_i is in registers: the tile takes S_{i+1}
                    ok = mbar_wait<kTest>(s_free, (uint32_t)i & 1u, abort_flag) && issue_s(i + 1);
                    if (!ok) break;
                }
                ok = mbar_wait<kTest>(p_full, (uint32_t)i & 1u, abort_flag);     // P_i is in TMEM, O rescaled if it had to be
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                const int s = i % S::kStages;
                const uint64_t dv = umma_desc(base + S::kOffKV + s * S::kStageBytes + S::kTileBytes, BK * 128);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)                       // 16 keys per step: 8 columns of P, two 8-key groups of V
                    umma_ts(tmem_o, tmem_p + 8 * kk, dv + (uint64_t)(2 * 1024 >> 4) * kk, idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(kv_empty(s));                                   // K_i and V_i have been read
                umma_commit(pv_done);                                       // P_i has been read, O holds steps 0..i
            }
        }
    } else {
        // ------------------------------------------------------------ softmax + output (thread = query row)
        const unsigned full = 0xffffffffu;
        const int r = warp * 32 + lane;                          // row of the tile, TMEM lane
        const int pos = start + tile * BQ + r;                   // position of this query
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const float sl2 = scale * kLog2e;
        float m_run = -INFINITY, l_run = 0.f;
        uint32_t sv[BK];
        bool ok = true;
        for (int i = 0; i < n_steps; ++i) {
            const int key0 = (j_lo + S::kPages * i) * kPageTokens;   // position of the step's first key
            ok = __all_sync(full, mbar_wait<kTest>(s_full, (uint32_t)i & 1u, abort_flag));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
#pragma unroll
            for (int c = 0; c < BK / 32; ++c) tmem_ld32(tmem_s + lane_off + 32 * c, sv + 32 * c);
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free);                  // S_i is in registers: the tile takes S_{i+1}
            const bool all_visible = (key0 + BK - 1 <= pos) && (window <= 0 || key0 > pos - window);
            if (!all_visible) {
#pragma unroll
                for (int c = 0; c < BK; ++c) {
                    const int key = key0 + c;
                    const bool vis = key <= pos && (window <= 0 || key > pos - window);
                    if (!vis) sv[c] = __float_as_uint(-INFINITY);
                }
            }
            float mx[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) mx[e] = -INFINITY;
#pragma unroll
            for (int c = 0; c < BK; c += 8) {
#pragma unroll
                for (int e = 0; e < 8; ++e) mx[e] = fmaxf(mx[e], __uint_as_float(sv[c + e]));
            }
            const float m_page = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                       fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7]))) * sl2;
            if (i == 0) {
                m_run = m_page;                                  // the first product overwrites O
            } else {
                const bool raise = m_page > m_run + kRaiseBy;    // also: the first visible key of a row
                if (__any_sync(full, raise)) {
                    // O may only be touched between products (rare after the first steps)
                    ok = __all_sync(full, mbar_wait<kTest>(pv_done, (uint32_t)(i - 1) & 1u, abort_flag));
                    if (!ok) break;
                    float corr = 1.0f;
                    if (raise) {
                        corr = fast_exp2(m_run - m_page);        // 0 when the row had seen nothing
                        m_run = m_page;
                        l_run *= corr;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
                    uint32_t ov[8];                              // few registers: the scores are live
#pragma unroll 1
                    for (int part = 0; part < HD / 8; ++part) {
                        tmem_ld8(tmem_o + lane_off + 8 * part, ov);
                        asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                        for (int d = 0; d < 8; ++d) ov[d] = __float_as_uint(__uint_as_float(ov[d]) * corr);
                        tmem_st8(tmem_o + lane_off + 8 * part, ov);
                    }
                }
            }
            const float m_use = m_run == -INFINITY ? 0.f : m_run;
            float l0 = 0.f, l1 = 0.f;
            // the row of P: BK bfloat16 as BK/2 packed columns (packed in place: the
            // pair of scores 2c, 2c+1 becomes word c).  Eight exponentials are issued
            // back to back before the first of them is used.
#pragma unroll
            for (int c = 0; c < BK / 2; c += 4) {
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) p[e] = fmaf(__uint_as_float(sv[2 * c + e]), sl2, -m_use);
#pragma unroll
                for (int e = 0; e < 8; ++e) p[e] = exp2_in_order(p[e]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    l0 += p[2 * e];
                    l1 += p[2 * e + 1];
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
                    sv[c + e] = *reinterpret_cast<uint32_t*>(&hh);   // the scores at and below this index are done with
                }
            }
            // P_i goes where P_{i-1} was: its product must have read it (it has, long ago,
            // unless the tensor pipe is the slower side)
            if (i > 0) {
                ok = __all_sync(full, mbar_wait<kTest>(pv_done, (uint32_t)(i - 1) & 1u, abort_flag));
                if (!ok) break;
            }
#pragma unroll
            for (int c = 0; c < BK / 64; ++c) tmem_st32(tmem_p + lane_off + 32 * c, sv + 32 * c);
            l_run += l0 + l1;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok) ok = __all_sync(full, mbar_wait<kTest>(pv_done, (uint32_t)(n_steps - 1) & 1u, abort_flag));
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            bf16* dst = out + (size_t)(q_begin + tile * BQ + r) * ldo + h * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                tmem_ld32(tmem_o + lane_off + 32 * c, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                if (r < rows_here) {
#pragma unroll
                    for (int piece = 0; piece < 4; ++piece) {
                        uint32_t o4[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(sv[8 * piece + 2 * q]) * inv,
                                                                      __uint_as_float(sv[8 * piece + 2 * q + 1]) * inv);
                            o4[q] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        *reinterpret_cast<uint4*>(dst + 32 * c + 8 * piece) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::);
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::);
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_s), "r"(kTmemCols));
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
// rows x cols bfloat16, `ld` elements between rows, boxes of 64 columns x box_rows.
int make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiled enc = encode_fn();
    if (!enc) return kErrUnsupported;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : kErrBadArgument;
}

template <int HD, bool kTest>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, bf16* out, int ldo, const int* block_table,
           int table_stride, const int* cu_seqlens, const int* slots, const int* start_pos, int B, int max_q_len,
           int n_heads, int n_kv, float scale, int window, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, kTest>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Shape<HD>::kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_heads, B, (max_q_len + BQ - 1) / BQ);
    return launch_chained(attention_prefill_tc_kernel<HD, kTest>, grid, dim3(kThreads), (size_t)Shape<HD>::kSmemBytes, stream,
                          map_q, map_kv, out, ldo, block_table, table_stride, cu_seqlens, slots, start_pos,
                          n_heads, n_kv, scale, window);
}
}  // namespace

GTG_API int gtg_attention_tcgen05_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// What this kernel serves: heads of 64 or 128 channels whose keys and values lie in
// one cache entry as [page][k|v][head][token][channel] (values right after the keys).
GTG_API int gtg_attention_tcgen05_supports(int hd) { return hd == 64 || hd == 128; }

// q: [n_tokens, ldq] with head h at columns h*hd; kc, vc: the entry's key and value
// bases; page_stride: elements between pages.  n_pages: pages of the entry's pool.
GTG_API int gtg_attention_prefill_tcgen05(const void* q, int ldq, int n_tokens, void* out, int ldo,
                                          const void* kc, const void* vc, long long page_stride, int n_pages,
                                          const int* block_table, int table_stride,
                                          const int* cu_seqlens, const int* slots, const int* start_pos,
                                          int B, int max_q_len, int n_heads, int n_kv, int hd,
                                          float scale, int window, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    if (hd != 64 && hd != 128) return kErrUnsupported;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0) return kErrBadArgument;
    if (ldq % 8 || ldo % 8 || ((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)kc % 16)) return kErrUnsupported;
    // keys then values of a page, contiguous: the layout the row arithmetic above assumes
    const long long kv_rows = 2LL * n_kv * kPageTokens;
    if (page_stride != kv_rows * hd || (const bf16*)vc != (const bf16*)kc + (long long)n_kv * kPageTokens * hd)
        return kErrUnsupported;
    if (B > 65535 || (max_q_len + BQ - 1) / BQ > 65535 || (long long)n_pages * kv_rows > 0x7fffffffLL) return kErrUnsupported;
    CUtensorMap map_q, map_kv;
    int st = make_map(&map_q, q, n_tokens, n_heads * hd, ldq, BQ);
    if (st != 0) return st;
    st = make_map(&map_kv, kc, (long long)n_pages * kv_rows, hd, hd, kPageTokens);
    if (st != 0) return st;
#define GTG_ARGS map_q, map_kv, (bf16*)out, ldo, block_table, table_stride, cu_seqlens, slots, start_pos, \
                 B, max_q_len, n_heads, n_kv, scale, window, stream
    if (g_test_waits) return hd == 64 ? launch<64, true>(GTG_ARGS) : launch<128, true>(GTG_ARGS);
    return hd == 64 ? launch<64, false>(GTG_ARGS) : launch<128, false>(GTG_ARGS);
#undef GTG_ARGS
}

// ---- test hook --------------------------------------------------------------
// For the test that makes bounded waits run out: while `test_waits` is set, every
// launch of this library takes the kTest form of its kernel (see Waits above): no
// asynchronous copy is issued, so no barrier completes, and every wait gives up
// after a thousand polls.  Such a kernel returns without a result and the status
// word reads non-zero; nothing faults and nothing hangs.  The kernels as they
// normally run are not touched by this.  The call also clears the status word.
GTG_API int gtg_attention_tcgen05_test_hooks(int test_waits) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    g_test_waits = test_waits != 0;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    return (int)e;
}

// bfloat16 attention over the paged cache on the warp-level tensor-core path.
//
//   attention_prefill: flash-style causal grouped-query attention for a batch of
//     prompts of unequal length.  One CTA per (64-query tile, query head,
//     sequence); it walks the sequence's cache pages (64 keys each) up to the
//     tile's last position with a streaming softmax in float.
//   attention_decode: one query per sequence.  One CTA per (split, key/value
//     head, sequence) serves the whole group of query heads that share the
//     key/value head (rows of one 16-row MMA tile), streams its share of the
//     pages through a cp.async ring of three pages (or four) and writes either the final
//     output or a partial (max, sum, accumulator) that attention_combine merges
//     in a fixed order.
//
// Scores are scaled after the dot product, masked by position (causal, optional
// window), and exponentiated with exp2 on log2(e)-scaled values; max, sum and
// the output accumulator are float (model/llama.go:1626-1660 for the formula).
// Head sizes 16..128 in steps of 16 are served by the 16/32/64/128-wide variant
// with zero-filled padding.
#include "mma_helpers.cuh"
#include <math.h>

namespace {

constexpr float kLog2e = 1.4426950408889634f;

// 2^x by the special-function unit; 2^(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// ============================================================= prefill
template <int DP>
__global__ void __launch_bounds__(128, DP <= 64 ? 4 : 1)
attention_prefill_kernel(const bf16* __restrict__ q, int ldq, bf16* __restrict__ out, int ldo,
                         const bf16* __restrict__ kc, const bf16* __restrict__ vc, long long page_stride,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                         const int* __restrict__ start_pos,
                         int n_heads, int n_kv, int hd, float scale, int window) {
    constexpr int CPR = DP / 8;                 // 16-byte chunks per row
    constexpr int TILE_BYTES = 64 * DP * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sK = sQ + TILE_BYTES;        // two stages
    const uint32_t sV = sK + 2 * TILE_BYTES;    // two stages

    const int b = blockIdx.z, h = blockIdx.y;
    const int tile = gridDim.x - 1 - blockIdx.x;          // longest tiles first
    const int q_begin = cu_seqlens[b];
    const int q_len = cu_seqlens[b + 1] - q_begin;
    if (tile * 64 >= q_len) return;
    const int start = start_pos[b];
    const int kvh = h / (n_heads / n_kv);
    const int* table = block_table + (size_t)slots[b] * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;

    const int rows_here = min(64, q_len - tile * 64);
    const int kv_total = start + q_len;                    // keys that exist after this step
    const int k_max = start + tile * 64 + rows_here - 1;   // last key any row of the tile sees
    int k_min = 0;
    if (window > 0) k_min = max(0, start + tile * 64 - window + 1);
    const int j_lo = k_min / kPageTokens, j_hi = k_max / kPageTokens;

    // ---- stage the query tile
    for (int id = tid; id < 64 * CPR; id += 128) {
        const int r = id / CPR, c = id % CPR;
        const bool ok = r < rows_here && c * 8 < hd;
        const bf16* src = ok ? q + (size_t)(q_begin + tile * 64 + r) * ldq + h * hd + c * 8 : q;
        cp_async16(sQ + swz_offset<DP>(r, c), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int stage, int j) {
        const size_t base = (size_t)table[j] * page_stride + (size_t)kvh * kPageTokens * hd;
        for (int id = tid; id < 64 * CPR; id += 128) {
            const int r = id / CPR, c = id % CPR;
            const bool ok = (j * kPageTokens + r) < kv_total && c * 8 < hd;
            const size_t off = ok ? base + (size_t)r * hd + c * 8 : 0;
            cp_async16(sK + stage * TILE_BYTES + swz_offset<DP>(r, c), kc + off, ok ? 16 : 0);
            cp_async16(sV + stage * TILE_BYTES + swz_offset<DP>(r, c), vc + off, ok ? 16 : 0);
        }
    };
    load_kv(0, j_lo);
    cp_async_commit();

    uint32_t qf[DP / 16][4];
    float o[DP / 8][4];
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_row[2] = {-INFINITY, -INFINITY};   // running max of scaled scores (log2 domain)
    float l_row[2] = {0.f, 0.f};               // this thread's share of the running sum
    const float sl2 = scale * kLog2e;
    const int pos0 = start + tile * 64 + warp * 16 + g;    // position of row g; row g+8 is pos0+8

    for (int j = j_lo, it = 0; j <= j_hi; ++j, ++it) {
        const int stage = it & 1;
        if (j + 1 <= j_hi) {
            load_kv(stage ^ 1, j + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int kk = 0; kk < DP / 16; ++kk) {
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + swz_offset<DP>(r, c));
            }
        }
        // ---- S = Q K^T for this warp's 16 rows and the page's 64 keys
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
        const uint32_t kbase = sK + stage * TILE_BYTES, vbase = sV + stage * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                uint32_t b0, b1, b2, b3;
                const int r = jj * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = kk * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b0, b1, b2, b3, kbase + swz_offset<DP>(r, c));
                mma_bf16_16816(s[jj * 2], qf[kk], b0, b1);
                mma_bf16_16816(s[jj * 2 + 1], qf[kk], b2, b3);
            }
        }
        // ---- mask (only the pages that cross this warp's diagonal or window edge),
        //      streaming softmax on raw scores: p = 2^(s * scale*log2e - m)
        const bool all_visible = (j * kPageTokens + kPageTokens - 1 <= pos0) &&
                                 (window <= 0 || j * kPageTokens > pos0 + 8 - window);
        if (!all_visible) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j * kPageTokens + i * 8 + t4 * 2 + (e & 1);
                    const int pos = pos0 + (e >> 1) * 8;
                    const bool ok = key <= pos && (window <= 0 || key > pos - window);
                    if (!ok) s[i][e] = -INFINITY;
                }
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[i][e]);
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_row[r], mx[r] * sl2);          // scale > 0: max commutes with it
            m_use[r] = m_new == -INFINITY ? 0.f : m_new;
            corr[r] = fast_exp2(m_row[r] - m_use[r]);
            m_row[r] = m_new;
            l_row[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = fast_exp2(fmaf(s[i][e], sl2, -m_use[e >> 1]));
                s[i][e] = p;
                l_row[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dd = 0; dd < DP / 16; ++dd) {
                uint32_t b0, b1, b2, b3;
                const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                const int c = dd * 2 + (lane >> 4);
                ldmatrix_x4_trans(b0, b1, b2, b3, vbase + swz_offset<DP>(r, c));
                mma_bf16_16816(o[dd * 2], pa, b0, b1);
                mma_bf16_16816(o[dd * 2 + 1], pa, b2, b3);
            }
        }
        __syncthreads();
    }

    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        if (row >= rows_here) continue;
        const float inv = l_row[r] > 0.f ? 1.0f / l_row[r] : 0.f;
        bf16* dst = out + (size_t)(q_begin + tile * 64 + row) * ldo + h * hd;
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
            const int d = i * 8 + t4 * 2;
            if (d < hd)
                *reinterpret_cast<__nv_bfloat162*>(dst + d) =
                    __floats2bfloat162_rn(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
        }
    }
}

// ============================================================== decode
// Pages in the ring of a decode block: three (two in flight while one is worked on) or
// four.  What the kernel reaches is set by how many blocks share an SM more than by how
// deep each one's ring is: with 16 KB pages (heads up to 64 channels) three stages let
// four blocks share an SM, and that beat three blocks of four stages at most batch
// sizes measured (and two blocks of six by far).  The exception is a batch that brings
// about one block per slot without any split: then the longest sequence's one block
// is what the step waits for, and the block with three pages in flight is the faster
// (`gtg_attention_decode_plan` picks).  Pages of 128 channels take 32 KB: three stages
// keep two blocks on an SM; two stages with three blocks were slower.
constexpr int kRingDefault = 3, kRingDeep = 4;
// Shared memory of a decode block: the queries, then the page ring (reused for the merge).
template <int DP, int STAGES>
constexpr int decode_smem_bytes() {
    constexpr int ring = STAGES * 2 * 64 * DP * 2;
    constexpr int merge = (4 * 16 * DP + 128) * 4;
    return 16 * DP * 2 + (ring > merge ? ring : merge);
}

// What a decode step's rotation-and-store kernel would do, done here instead (all
// null: q arrives rotated and the new keys and values are in the cache already).
//   cos_sin: (cos, sin) [B][hd/2] of each sequence's new position: the queries are
//            rotated in shared memory after they arrive, the new key before it is used.
//   k_new, v_new: the new token's keys and values as the projection wrote them, rows
//            of `ldq` elements (n_kv heads of hd channels each).  The block that
//            holds the sequence's newest page puts them (the key rotated) into its
//            staged copy of that page, and one block per key/value head also into
//            the cache (kc_w, vc_w), for the steps to come.
struct DecodeRope {
    const float2* cos_sin;
    const bf16* k_new;
    const bf16* v_new;
    bf16* kc_w;
    bf16* vc_w;
};
// (a, b) at rotary frequency i -> (a cos - b sin, a sin + b cos), as rope_kv_store computes it
__device__ __forceinline__ void rotate_pair(float a, float b, float2 cs, bf16& ra, bf16& rb) {
    ra = __float2bfloat16_rn(a * cs.x - b * cs.y);
    rb = __float2bfloat16_rn(a * cs.y + b * cs.x);
}

// Partials: for each (sequence, query head, split): DP floats of unnormalised
// output, then the running max (log2 domain) and the running sum.
template <int DP, int STAGES>
__global__ void __launch_bounds__(128)
attention_decode_kernel(const bf16* __restrict__ q, int ldq, bf16* __restrict__ out, int ldo,
                        const bf16* __restrict__ kc, const bf16* __restrict__ vc, long long page_stride,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ slots, const int* __restrict__ positions,
                        int n_heads, int n_kv, int hd, float scale, int window,
                        int n_splits, float* __restrict__ part_o, float* __restrict__ part_ml,
                        const DecodeRope rope, int chunk_pages) {
    chain_release();
    constexpr int kDecodeStages = STAGES;
    constexpr int CPR = DP / 8;
    constexpr int TILE_BYTES = 64 * DP * 2;
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t sQ = smem_u32(smem);                       // 16 x DP bf16
    const uint32_t sKV = sQ + 16 * DP * 2;                    // kDecodeStages x (K page, V page)
    float* merge = reinterpret_cast<float*>(smem + 16 * DP * 2);   // reused after the page loop

    const int split = blockIdx.x, b = blockIdx.z;
    const int group = n_heads / n_kv;
    const int tiles_per_kv = (group + 15) / 16;
    const int kvh = blockIdx.y / tiles_per_kv;
    const int h0 = kvh * group + (blockIdx.y % tiles_per_kv) * 16;   // first query head of this CTA
    const int rows = min(16, kvh * group + group - h0);              // query heads served here
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;

    const int pos = positions[b];
    const int* table = block_table + (size_t)slots[b] * table_stride;
    const int k_min = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int p_first = k_min / kPageTokens, p_last = pos / kPageTokens;
    const int n_pages = p_last - p_first + 1;
    // With `chunk_pages` (the pages one split was planned to take) a sequence is cut into
    // as many equal parts as give parts of about that size, at most n_splits: a short
    // sequence costs few blocks of full size instead of as many small ones as the
    // longest.  With chunk_pages 0 every sequence is cut into n_splits parts.
    const int my_splits = chunk_pages > 0 ? min(n_splits, (n_pages + chunk_pages - 1) / chunk_pages) : n_splits;
    const int per_split = (n_pages + my_splits - 1) / my_splits;
    const int p_begin = p_first + split * per_split;
    const int p_end = split < my_splits ? min(p_last + 1, p_begin + per_split) : p_begin;    // exclusive
    if (n_splits > 1 && p_begin >= p_end) {
        // nothing of this sequence falls to this split: say so (the merge passes over it) and leave
        chain_wait();
        for (int r = threadIdx.x; r < rows; r += blockDim.x) {
            const size_t pidx = ((size_t)b * n_heads + h0 + r) * n_splits + split;
            part_ml[pidx * 2] = -INFINITY;
            part_ml[pidx * 2 + 1] = 0.f;
        }
        return;
    }

    auto load_page = [&](int stage, int p) {
        const size_t base = (size_t)table[p] * page_stride + (size_t)kvh * kPageTokens * hd;
        const uint32_t dk = sKV + stage * STAGE_BYTES, dv = dk + TILE_BYTES;
        for (int id = tid; id < 64 * CPR; id += 128) {
            const int r = id / CPR, c = id % CPR;
            const bool ok = (p * kPageTokens + r) <= pos && c * 8 < hd;
            const size_t off = ok ? base + (size_t)r * hd + c * 8 : 0;
            cp_async16(dk + swz_offset<DP>(r, c), kc + off, ok ? 16 : 0);
            cp_async16(dv + swz_offset<DP>(r, c), vc + off, ok ? 16 : 0);
        }
    };
    // Pages before the newest one were completed by earlier steps: their copies may
    // start while the kernels before this one (the projection, the rotation that
    // writes the newest key and value) are still running.  Positions, slots and the
    // block table were written before the projection began.  When this kernel adds
    // the new token itself, the newest page holds nothing newer than the step before
    // either (its row for the new token is replaced below) and goes with the others.
    const bool adds_token = rope.k_new != nullptr;
#pragma unroll
    for (int s = 0; s < kDecodeStages - 1; ++s)
        if (p_begin + s < p_end && (p_begin + s < p_last || adds_token)) load_page(s, p_begin + s);
    chain_wait();
    // ---- queries of the group (rows beyond `rows` are zero)
    for (int id = tid; id < 16 * CPR; id += 128) {
        const int r = id / CPR, c = id % CPR;
        const bool ok = r < rows && c * 8 < hd;
        const bf16* src = ok ? q + (size_t)b * ldq + (h0 + r) * hd + c * 8 : q;
        cp_async16(sQ + swz_offset<DP>(r, c), src, ok ? 16 : 0);
    }
#pragma unroll
    for (int s = 0; s < kDecodeStages - 1; ++s) {
        if (p_begin + s < p_end && p_begin + s == p_last && !adds_token) load_page(s, p_last);
        cp_async_commit();
    }

    uint32_t qf[DP / 16][4];
    float o[DP / 8][4];
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_row[2] = {-INFINITY, -INFINITY};
    float l_row[2] = {0.f, 0.f};
    const float sl2 = scale * kLog2e;

    for (int p = p_begin, it = 0; p < p_end; ++p, ++it) {
        cp_async_wait<kDecodeStages - 2>();
        __syncthreads();
        {
            const int nxt = p + kDecodeStages - 1;
            if (nxt < p_end) load_page((it + kDecodeStages - 1) % kDecodeStages, nxt);
            cp_async_commit();
        }
        const int half = hd >> 1;
        if (it == 0) {
            if (rope.cos_sin != nullptr) {                    // the queries arrived unrotated
                for (int id = tid; id < rows * half; id += 128) {
                    const int r = id / half, i = id - r * half;
                    bf16* pa = reinterpret_cast<bf16*>(smem + swz_offset<DP>(r, i >> 3)) + (i & 7);
                    bf16* pb = reinterpret_cast<bf16*>(smem + swz_offset<DP>(r, (i + half) >> 3)) + ((i + half) & 7);
                    rotate_pair(__bfloat162float(*pa), __bfloat162float(*pb), rope.cos_sin[(size_t)b * half + i], *pa, *pb);
                }
                __syncthreads();
            }
#pragma unroll
            for (int kk = 0; kk < DP / 16; ++kk) {
                const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], sQ + swz_offset<DP>(r, c));
            }
        }
        if (adds_token && p == p_last) {
            // the new token's key (rotated) and value: into the staged page, and once per
            // key/value head into the cache
            const int rr = pos % kPageTokens;
            unsigned char* kt = smem + 16 * DP * 2 + (it % kDecodeStages) * STAGE_BYTES;
            unsigned char* vt = kt + TILE_BYTES;
            const bool writer = rope.kc_w != nullptr && blockIdx.y % tiles_per_kv == 0;
            const size_t goff = (size_t)table[p_last] * page_stride + ((size_t)kvh * kPageTokens + rr) * hd;
            const bf16* ksrc = rope.k_new + (size_t)b * ldq + kvh * hd;
            const bf16* vsrc = rope.v_new + (size_t)b * ldq + kvh * hd;
            for (int i = tid; i < half; i += 128) {
                bf16 ka = ksrc[i], kb = ksrc[i + half];
                if (rope.cos_sin != nullptr)
                    rotate_pair(__bfloat162float(ka), __bfloat162float(kb), rope.cos_sin[(size_t)b * half + i], ka, kb);
                const bf16 va = vsrc[i], vb = vsrc[i + half];
                const uint32_t oa = swz_offset<DP>(rr, i >> 3) + (i & 7) * 2;
                const uint32_t ob = swz_offset<DP>(rr, (i + half) >> 3) + ((i + half) & 7) * 2;
                *reinterpret_cast<bf16*>(kt + oa) = ka;
                *reinterpret_cast<bf16*>(kt + ob) = kb;
                *reinterpret_cast<bf16*>(vt + oa) = va;
                *reinterpret_cast<bf16*>(vt + ob) = vb;
                if (writer) {
                    rope.kc_w[goff + i] = ka;
                    rope.kc_w[goff + i + half] = kb;
                    rope.vc_w[goff + i] = va;
                    rope.vc_w[goff + i + half] = vb;
                }
            }
            __syncthreads();
        }
        const uint32_t kbase = sKV + (it % kDecodeStages) * STAGE_BYTES, vbase = kbase + TILE_BYTES;
        // this warp's 16 keys of the page: S[16 heads x 16 keys]
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk) {
            uint32_t b0, b1, b2, b3;
            const int r = warp * 16 + (lane & 7) + (lane >> 4) * 8;
            const int c = kk * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b0, b1, b2, b3, kbase + swz_offset<DP>(r, c));
            mma_bf16_16816(s[0], qf[kk], b0, b1);
            mma_bf16_16816(s[1], qf[kk], b2, b3);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = p * kPageTokens + warp * 16 + i * 8 + t4 * 2 + (e & 1);
                const bool ok = key <= pos && key >= k_min;
                const float v = ok ? s[i][e] * sl2 : -INFINITY;
                s[i][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_row[r], mx[r]);
            m_use[r] = m_new == -INFINITY ? 0.f : m_new;
            corr[r] = exp2f(m_row[r] - m_use[r]);
            m_row[r] = m_new;
            l_row[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[i][e] - m_use[e >> 1]);
                s[i][e] = pv;
                l_row[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dd = 0; dd < DP / 16; ++dd) {
            uint32_t b0, b1, b2, b3;
            const int r = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int c = dd * 2 + (lane >> 4);
            ldmatrix_x4_trans(b0, b1, b2, b3, vbase + swz_offset<DP>(r, c));
            mma_bf16_16816(o[dd * 2], pa, b0, b1);
            mma_bf16_16816(o[dd * 2 + 1], pa, b2, b3);
        }
    }
    cp_async_wait<0>();
    __syncthreads();      // every warp is done with the ring: reuse it for the merge

    // ---- merge the four warps (each saw a quarter of every page) in warp order
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    }
    float* mo = merge;                      // [4 warps][16 rows][DP]
    float* mm = merge + 4 * 16 * DP;        // [4][16] max
    float* ml = mm + 64;                    // [4][16] sum
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + r * 8;
        if (t4 == 0) { mm[warp * 16 + row] = m_row[r]; ml[warp * 16 + row] = l_row[r]; }
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
            const int d = i * 8 + t4 * 2;
            mo[(warp * 16 + row) * DP + d] = o[i][r * 2];
            mo[(warp * 16 + row) * DP + d + 1] = o[i][r * 2 + 1];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < rows * DP; idx += 128) {
        const int row = idx / DP, d = idx % DP;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 16 + row]);
        const float Mu = M == -INFINITY ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(mm[w * 16 + row] - Mu);
            acc += f * mo[(w * 16 + row) * DP + d];
            L += f * ml[w * 16 + row];
        }
        const int head = h0 + row;
        if (n_splits == 1) {
            if (d < hd) out[(size_t)b * ldo + head * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t pidx = ((size_t)b * n_heads + head) * n_splits + split;
            part_o[pidx * DP + d] = acc;
            if (d == 0) { part_ml[pidx * 2] = M; part_ml[pidx * 2 + 1] = L; }
        }
    }
}

constexpr int kCombineAtOnce = 16;

template <int DP>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, int ldo, int n_heads, int hd, int n_splits) {
    chain_release();
    chain_wait();
    const int bh = blockIdx.x;                 // sequence * n_heads + head
    const int b = bh / n_heads, head = bh % n_heads;
    const int d = threadIdx.x;
    if (d >= hd) return;
    if (n_splits <= kCombineAtOnce) {
        // Few splits: everything this thread reads is asked for at once (one trip to the
        // L2 instead of two in a row), then added up in the order of the loop below.
        float ms[kCombineAtOnce], ls[kCombineAtOnce], os[kCombineAtOnce];
#pragma unroll
        for (int s = 0; s < kCombineAtOnce; ++s) {
            ms[s] = -INFINITY;
            ls[s] = os[s] = 0.f;
            if (s < n_splits) {
                const size_t pidx = (size_t)bh * n_splits + s;
                const float2 ml = *reinterpret_cast<const float2*>(part_ml + pidx * 2);
                ms[s] = ml.x;
                ls[s] = ml.y;
                os[s] = part_o[pidx * DP + d];
            }
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < kCombineAtOnce; ++s) M = fmaxf(M, ms[s]);
        const float Mu = M == -INFINITY ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int s = 0; s < kCombineAtOnce; ++s) {
            if (ms[s] == -INFINITY) continue;      // a split without keys wrote no sums (what was read for it is not used)
            const float f = exp2f(ms[s] - Mu);
            acc += f * os[s];
            L += f * ls[s];
        }
        out[(size_t)b * ldo + head * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        return;
    }
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[((size_t)bh * n_splits + s) * 2]);
    const float Mu = M == -INFINITY ? 0.f : M;
    float acc = 0.f, L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const size_t pidx = (size_t)bh * n_splits + s;
        const float m = part_ml[pidx * 2];
        if (m == -INFINITY) continue;              // a split without keys wrote no sums
        const float f = exp2f(m - Mu);
        acc += f * part_o[pidx * DP + d];
        L += f * part_ml[pidx * 2 + 1];
    }
    out[(size_t)b * ldo + head * hd + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

int padded_head_dim(int hd) {
    if (hd <= 0 || hd % 16 != 0 || hd > 128) return 0;
    if (hd <= 16) return 16;
    if (hd <= 32) return 32;
    if (hd <= 64) return 64;
    return 128;
}

template <int DP>
int launch_prefill(const bf16* q, int ldq, bf16* out, int ldo, const bf16* kc, const bf16* vc,
                   long long page_stride, const int* block_table, int table_stride,
                   const int* cu_seqlens, const int* slots, const int* start_pos,
                   int B, int max_q_len, int n_heads, int n_kv, int hd, float scale, int window,
                   cudaStream_t stream) {
    static bool configured = false;
    const int smem = 5 * 64 * DP * 2;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_q_len + 63) / 64, n_heads, B);
    attention_prefill_kernel<DP><<<grid, 128, smem, stream>>>(q, ldq, out, ldo, kc, vc, page_stride,
        block_table, table_stride, cu_seqlens, slots, start_pos, n_heads, n_kv, hd, scale, window);
    return launch_status();
}

template <int DP, int STAGES>
int launch_decode_ring(const bf16* q, int ldq, bf16* out, int ldo, const bf16* kc, const bf16* vc,
                       long long page_stride, const int* block_table, int table_stride,
                       const int* slots, const int* positions, int B, int n_heads, int n_kv, int hd,
                       float scale, int window, int n_splits, float* part_o, float* part_ml,
                       cudaStream_t stream, const DecodeRope rope, int chunk_pages) {
    static bool configured = false;
    const int smem = decode_smem_bytes<DP, STAGES>();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<DP, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int group = n_heads / n_kv;
    dim3 grid(n_splits, n_kv * ((group + 15) / 16), B);
    int st = launch_chained(attention_decode_kernel<DP, STAGES>, grid, dim3(128), smem, stream, q, ldq, out, ldo, kc, vc,
                            page_stride, block_table, table_stride, slots, positions, n_heads, n_kv, hd, scale,
                            window, n_splits, part_o, part_ml, rope, n_splits > 1 ? chunk_pages : 0);
    if (st != 0 || n_splits == 1) return st;
    return launch_chained(attention_combine_kernel<DP>, dim3(B * n_heads), dim3(DP), 0, stream,
                          (const float*)part_o, (const float*)part_ml, out, ldo, n_heads, hd, n_splits);
}

// ring_pages: kRingDeep where the plan asked for it (heads up to 64 channels), else the default.
template <int DP>
int launch_decode(const bf16* q, int ldq, bf16* out, int ldo, const bf16* kc, const bf16* vc,
                  long long page_stride, const int* block_table, int table_stride,
                  const int* slots, const int* positions, int B, int n_heads, int n_kv, int hd,
                  float scale, int window, int n_splits, float* part_o, float* part_ml,
                  cudaStream_t stream, const DecodeRope rope, int chunk_pages, int ring_pages) {
    if constexpr (DP <= 64) {
        if (ring_pages == kRingDeep)
            return launch_decode_ring<DP, kRingDeep>(q, ldq, out, ldo, kc, vc, page_stride, block_table, table_stride, slots,
                                                     positions, B, n_heads, n_kv, hd, scale, window, n_splits, part_o,
                                                     part_ml, stream, rope, chunk_pages);
    }
    return launch_decode_ring<DP, kRingDefault>(q, ldq, out, ldo, kc, vc, page_stride, block_table, table_stride, slots,
                                                positions, B, n_heads, n_kv, hd, scale, window, n_splits, part_o, part_ml,
                                                stream, rope, chunk_pages);
}
}  // namespace

// Head sizes the tiled bfloat16 kernels serve (others go to the one-warp-per-row kernel).
GTG_API int gtg_attention_bf16_supports(int hd) { return padded_head_dim(hd) != 0; }

// ---- into how many blocks to split the keys of one (sequence, key/value head)
// How many decode blocks the current device holds at once: what the occupancy
// calculator says for this kernel's registers and shared memory, times the
// device's multiprocessors.  Asked once per (device, head size).
template <int DP, int STAGES>
static int decode_block_slots() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] == 0) {
        constexpr int smem = decode_smem_bytes<DP, STAGES>();
        int per_sm = 0, sms = 0;
        if (cudaFuncSetAttribute(attention_decode_kernel<DP, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<DP, STAGES>, 128, smem) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        cached[dev] = sms * (per_sm > 0 ? per_sm : 1);
    }
    return cached[dev];
}

// Into how many blocks to split the keys of a (sequence, key/value head), for a
// batch whose longest sequence has max_kv_len keys and whose sequences have
// total_kv_len keys together (0: take all B as long as the longest).  A block
// costs a fixed latency (its first pages' round trip, the merge of its warps, its
// partial result) and then a page time each; blocks run in waves of what the
// device holds at once.  The estimate below is the time of blocks of `chunk`
// pages (side by side while the device holds them all, their times added up over
// its slots beyond that), or the time the memory needs for all keys, whichever
// is longer; the chunk with the least estimate wins.  A sequence then takes
// ceil(its pages / chunk) splits (the kernel works that out from its length), so
// the choice depends on the batch's lengths and the window only, never on the
// data.  A layer with a window reads the pages its window spans.  Returns the
// split count for the longest sequence (1 to 64), or a negative error code;
// *chunk_pages: the pages a split takes.  A sequence that has outgrown
// splits x chunk pages (a recorded step replayed while its sequences grow) is cut
// into `splits` parts of more pages each: the plan is a matter of speed only.
GTG_API int gtg_attention_decode_plan(int B, int n_heads, int n_kv, int hd, int max_kv_len, long long total_kv_len,
                                      int window, int* chunk_pages, int* ring_pages) {
    if (chunk_pages) *chunk_pages = 0;
    if (ring_pages) *ring_pages = kRingDefault;
    if (B <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0) return kErrBadArgument;
    int slots = 0, slots_deep = 0;
    const int dp = padded_head_dim(hd);
    switch (dp) {
        case 16: slots = decode_block_slots<16, kRingDefault>(); slots_deep = decode_block_slots<16, kRingDeep>(); break;
        case 32: slots = decode_block_slots<32, kRingDefault>(); slots_deep = decode_block_slots<32, kRingDeep>(); break;
        case 64: slots = decode_block_slots<64, kRingDefault>(); slots_deep = decode_block_slots<64, kRingDeep>(); break;
        case 128: slots = decode_block_slots<128, kRingDefault>(); break;
        default: return kErrUnsupported;
    }
    if (slots <= 0) return 1;
    const long long units = (long long)n_kv * ((n_heads / n_kv + 15) / 16);      // blocks per split of one sequence
    // The deeper ring, for the batch that fills the device about once with one block per
    // (sequence, head group): more blocks than the deep form's slots (below that, cutting
    // the sequences finer over the default form's many slots wins) and up to a fifth
    // more than the default form's (beyond, the blocks queue and their number per SM
    // counts again).  Measured at 32 head groups over prompts of 128 to 2,048 tokens:
    // the default form wins at 4, 12, 24, 32 and 48 sequences by 1 to 7 %, the deep
    // form at 16 and 20 by 6 %.
    int ring = kRingDefault;
    if (slots_deep > 0 && (long long)B * units > slots_deep && (long long)B * units <= slots + slots / 5) {
        ring = kRingDeep;
        slots = slots_deep;
    }
    if (ring_pages) *ring_pages = ring;
    auto span = [&](long long keys) {                                              // pages that hold `keys` keys
        long long pages = (keys + kPageTokens - 1) / kPageTokens;
        if (window > 0 && window < keys) {
            const long long w = (window + kPageTokens - 2) / kPageTokens + 1;      // `window` consecutive keys touch at most this many
            if (w < pages) pages = w;
        }
        return pages < 1 ? 1 : pages;
    };
    const int max_pages = (int)span(max_kv_len > 1 ? max_kv_len : 1);
    long long mean_keys = total_kv_len > 0 ? (total_kv_len + B - 1) / B : max_kv_len;
    if (mean_keys > max_kv_len) mean_keys = max_kv_len;
    const double mean_pages = (double)span(mean_keys > 1 ? mean_keys : 1);
    // measured on a B200: about 3.5 us before a block's first page is in use; a block
    // keeps all but one stage of its ring in flight over that latency (two pages:
    // 1.75 us a page; three: 1.17); the memory's own time for all keys, once enough
    // blocks run to saturate it
    const double kFixedUs = 3.5, kMergeUs = 3.0, kBytesPerUs = 6.0e6;
    const double kPageUs = kFixedUs / (ring - 1);
    const double page_bytes = 2.0 * kPageTokens * dp * 2;
    const double memory_us = (double)B * mean_pages * units * page_bytes / kBytesPerUs;
    int best_chunk = max_pages;
    double best = 1e30;
    for (int chunk = 1; chunk <= max_pages; ++chunk) {
        const int splits = (max_pages + chunk - 1) / chunk;
        if (splits > 64) continue;
        // blocks of the batch: a sequence of the mean length takes about mean / chunk + 1/2 splits
        const double per_seq = mean_pages >= max_pages ? (double)splits
                             : mean_pages / chunk < 1.0 ? 1.0 : (mean_pages / chunk + 0.5);
        const double blocks = (double)B * units * per_seq;
        const int longest = (max_pages + splits - 1) / splits;                     // pages of the longest sequence's splits
        const double longest_us = kFixedUs + kPageUs * longest;
        // What the device holds at once runs side by side.  Beyond that: blocks of one
        // length run in whole waves; blocks of many lengths (the long ones started first)
        // fill the slots evenly, their times add up over the slots and the last ends half
        // a typical block after the rest -- unless one long block outlasts all that.
        double us;
        if (blocks <= slots) {
            us = longest_us;
        } else if (mean_pages >= max_pages) {
            us = (double)(((long long)blocks + slots - 1) / slots) * longest_us;
        } else {
            const double typical_us = kFixedUs + kPageUs * (mean_pages < chunk ? mean_pages : chunk);
            us = (blocks * kFixedUs + kPageUs * B * units * mean_pages) / slots + 0.5 * typical_us;
            if (us < longest_us) us = longest_us;
        }
        if (us < memory_us) us = memory_us;
        if (splits > 1) us += kMergeUs;
        if (us < best - 1e-9) { best = us; best_chunk = chunk; }
    }
    if (chunk_pages) *chunk_pages = best_chunk;
    return (max_pages + best_chunk - 1) / best_chunk;
}

// Floats of scratch a decode call needs: (part_o, part_ml) for `n_splits` > 1.
GTG_API long long gtg_attention_decode_scratch_floats(int B, int n_heads, int hd, int n_splits) {
    const int dp = padded_head_dim(hd);
    if (dp == 0 || n_splits <= 1) return 0;
    return (long long)B * n_heads * n_splits * (dp + 2);
}

GTG_API int gtg_attention_prefill_bf16(const void* q, int ldq, void* out, int ldo,
                                       const void* kc, const void* vc, long long page_stride,
                                       const int* block_table, int table_stride,
                                       const int* cu_seqlens, const int* slots, const int* start_pos,
                                       int B, int max_q_len, int n_heads, int n_kv, int hd,
                                       float scale, int window, cudaStream_t stream) {
    if (B <= 0 || max_q_len <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || ldq % 8 != 0 || ldo % 2 != 0) return kErrBadArgument;
    if (n_heads > 65535 || B > 65535) return kErrUnsupported;
#define GTG_ARGS (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kc, (const bf16*)vc, page_stride, \
        block_table, table_stride, cu_seqlens, slots, start_pos, B, max_q_len, n_heads, n_kv, hd, scale, window, stream
    switch (padded_head_dim(hd)) {
        case 16: return launch_prefill<16>(GTG_ARGS);
        case 32: return launch_prefill<32>(GTG_ARGS);
        case 64: return launch_prefill<64>(GTG_ARGS);
        case 128: return launch_prefill<128>(GTG_ARGS);
        default: return kErrUnsupported;
    }
#undef GTG_ARGS
}

// For both decode entry points: with `chunk_pages` (0, or what gtg_attention_decode_plan
// gave) a sequence is cut into as many equal parts as give parts of about that many
// pages, at most n_splits, instead of into n_splits parts whatever its length.
// Blocks are handed out sequence by sequence in batch order: a caller whose
// sequences differ much in length does well to put the long ones first.
//
// Decode attention that also does what rope_kv_store does for a decode step (see
// DecodeRope): q, k_new and v_new are the unrotated columns of the projection's
// output (rows of ldq elements); cos_sin float [B][hd/2][2] or null for no rotation;
// k_new null if this layer adds nothing to the cache (then v_new is ignored);
// `store` 0 keeps the new token out of the cache (it is still attended to).
GTG_API int gtg_attention_decode_rope_bf16(const void* q, int ldq, void* out, int ldo,
                                           void* kc, void* vc, long long page_stride,
                                           const int* block_table, int table_stride,
                                           const int* slots, const int* positions,
                                           int B, int n_heads, int n_kv, int hd, float scale, int window,
                                           int n_splits, float* scratch, const float* cos_sin,
                                           const void* k_new, const void* v_new, int store,
                                           int chunk_pages, int ring_pages, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || ldq % 8 != 0 || n_splits < 1) return kErrBadArgument;
    if (k_new != nullptr && v_new == nullptr) return kErrBadArgument;
    const int dp = padded_head_dim(hd);
    if (dp == 0 || B > 65535 || n_splits > 65535) return kErrUnsupported;
    if (n_splits > 1 && scratch == nullptr) return kErrBadArgument;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)B * n_heads * n_splits * dp : nullptr;
    DecodeRope rope = {};
    rope.cos_sin = (const float2*)cos_sin;
    rope.k_new = (const bf16*)k_new;
    rope.v_new = (const bf16*)v_new;
    if (k_new != nullptr && store) { rope.kc_w = (bf16*)kc; rope.vc_w = (bf16*)vc; }
#define GTG_ARGS (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kc, (const bf16*)vc, page_stride, \
        block_table, table_stride, slots, positions, B, n_heads, n_kv, hd, scale, window, n_splits, part_o, part_ml, \
        stream, rope, chunk_pages, ring_pages
    switch (dp) {
        case 16: return launch_decode<16>(GTG_ARGS);
        case 32: return launch_decode<32>(GTG_ARGS);
        case 64: return launch_decode<64>(GTG_ARGS);
        case 128: return launch_decode<128>(GTG_ARGS);
        default: return kErrUnsupported;
    }
#undef GTG_ARGS
}

GTG_API int gtg_attention_decode_bf16(const void* q, int ldq, void* out, int ldo,
                                      const void* kc, const void* vc, long long page_stride,
                                      const int* block_table, int table_stride,
                                      const int* slots, const int* positions,
                                      int B, int n_heads, int n_kv, int hd, float scale, int window,
                                      int n_splits, float* scratch, int chunk_pages, int ring_pages,
                                      cudaStream_t stream) {
    if (B <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || ldq % 8 != 0 || n_splits < 1) return kErrBadArgument;
    const int dp = padded_head_dim(hd);
    if (dp == 0 || B > 65535 || n_splits > 65535) return kErrUnsupported;
    if (n_splits > 1 && scratch == nullptr) return kErrBadArgument;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)B * n_heads * n_splits * dp : nullptr;
#define GTG_ARGS (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)kc, (const bf16*)vc, page_stride, \
        block_table, table_stride, slots, positions, B, n_heads, n_kv, hd, scale, window, n_splits, part_o, part_ml, stream, \
        DecodeRope{}, chunk_pages, ring_pages
    switch (dp) {
        case 16: return launch_decode<16>(GTG_ARGS);
        case 32: return launch_decode<32>(GTG_ARGS);
        case 64: return launch_decode<64>(GTG_ARGS);
        case 128: return launch_decode<128>(GTG_ARGS);
        default: return kErrUnsupported;
    }
#undef GTG_ARGS
}

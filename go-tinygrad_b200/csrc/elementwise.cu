// Bandwidth-bound kernels around the matrix products: embedding gather, the
// residual add fused with RMSNorm, SwiGLU, the rotary table of a step and the
// rotation of queries and keys fused with the write into the paged cache.
// Each is templated on the activation type (float for the 32-bit path,
// __nv_bfloat16 for the serving path); sums, the reciprocal root, the rotation
// and the residual stream are float in both.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[n,:] = table[tokens[n],:] widened to float (the residual stream).  No
// scaling (model/inference_helpers.go:9-34).  Token ids are validated by the
// host; an id outside the table is clamped so the kernel never reads outside.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ out, int H, int V) {
    chain_wait();        // the step's metadata is written here or just before: nothing later may start early
    chain_release();
    const int n = blockIdx.x;
    int tok = tokens[n];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    const T* src = table + (size_t)tok * H;
    float* dst = out + (size_t)n * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

GTG_API int gtg_embed(int dtype, const int* tokens, const void* table, float* out,
                      int N, int H, int V, cudaStream_t stream) {
    int st = 0;
    if (N <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == 0) st = launch_chained(embed_kernel<float>, dim3(N), dim3(threads), 0, stream, tokens, (const float*)table, out, H, V);
    else if (dtype == 1) st = launch_chained(embed_kernel<bf16>, dim3(N), dim3(threads), 0, stream, tokens, (const bf16*)table, out, H, V);
    else return kErrBadArgument;
    return st;
}

// ------------------------------------------------- residual add + RMSNorm
// x = residual[r,:] (+ pending[r,:]);  out[i,:] = weight * x * (1/sqrt(mean(x^2)+eps))
// with r = rows ? rows[i] : i.  Without `rows` the sum is written back to the
// residual stream.  eps is added to the mean inside the root, and the product
// is (w*x)*s (backends/simd/vec.go:72-85).
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ pending,
                                   const float* __restrict__ weight, float eps,
                                   T* __restrict__ out, const int* __restrict__ rows, int H) {
    chain_release();
    chain_wait();
    extern __shared__ float smem[];
    float* row = smem;          // H floats
    float* scratch = smem + H;  // 33 floats
    const int i_out = blockIdx.x;
    const int r = rows ? rows[i_out] : i_out;
    float* res = residual + (size_t)r * H;
    const T* pen = pending ? pending + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = res[i];
        if (pen) {
            x += to_f32<T>(pen[i]);
            if (!rows) res[i] = x;
        }
        row[i] = x;
        ss += x * x;
    }
    const float total = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(total / (float)H + eps);
    T* o = out + (size_t)i_out * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f32<T>((weight[i] * row[i]) * s);
}

// The same for bfloat16 rows whose width is a multiple of 8 and at most 8192:
// every thread owns 8 consecutive channels, moved with 16- and 32-byte accesses
// and kept in registers between the sum of squares and the scaling.
__global__ void __launch_bounds__(1024)
add_rmsnorm_bf16_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ pending,
                            const float* __restrict__ weight, float eps, bf16* __restrict__ out,
                            const int* __restrict__ rows, int H) {
    chain_release();
    chain_wait();
    __shared__ float scratch[33];
    const int i_out = blockIdx.x;
    const int r = rows ? rows[i_out] : i_out;
    const int c = threadIdx.x * 8;
    const bool active = c < H;
    float x[8];
    float w[8];
    float ss = 0.f;
    if (active) {
        const float4* wp = reinterpret_cast<const float4*>(weight + c);
        const float4 w0 = wp[0], w1 = wp[1];
        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
        float4* rp = reinterpret_cast<float4*>(residual + (size_t)r * H + c);
        const float4 a = rp[0], b = rp[1];
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        if (pending) {
            const uint4 p = *reinterpret_cast<const uint4*>(pending + (size_t)r * H + c);
            const __nv_bfloat162* ph = reinterpret_cast<const __nv_bfloat162*>(&p);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(ph[j]);
                x[2 * j] += f.x;
                x[2 * j + 1] += f.y;
            }
            if (!rows) {
                rp[0] = make_float4(x[0], x[1], x[2], x[3]);
                rp[1] = make_float4(x[4], x[5], x[6], x[7]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    }
    const float total = block_sum(ss, scratch);
    const float s = 1.0f / sqrtf(total / (float)H + eps);
    if (active) {
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            oh[j] = __floats2bfloat162_rn((w[2 * j] * x[2 * j]) * s, (w[2 * j + 1] * x[2 * j + 1]) * s);
        *reinterpret_cast<uint4*>(out + (size_t)i_out * H + c) = o;
    }
}

GTG_API int gtg_add_rmsnorm(int dtype, float* residual, const void* pending, const float* weight,
                            float eps, void* out, const int* rows, int R, int H,
                            cudaStream_t stream) {
    int st = 0;
    if (R <= 0) return 0;
    if (dtype == 1 && H % 8 == 0 && H <= 8192 && ((uintptr_t)residual % 16) == 0 && ((uintptr_t)out % 16) == 0 &&
        ((uintptr_t)weight % 16) == 0 && ((uintptr_t)pending % 16) == 0) {
        int t = ((H / 8) + 31) / 32 * 32;
        st = launch_chained(add_rmsnorm_bf16_vec_kernel, dim3(R), dim3(t), 0, stream, residual, (const bf16*)pending, weight, eps, (bf16*)out, rows, H);
        return st;
    }
    int threads = 32;
    while (threads < 1024 && threads * 4 < H) threads *= 2;
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return kErrUnsupported;
    cudaError_t e;
    if (dtype == 0) {
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        st = launch_chained(add_rmsnorm_kernel<float>, dim3(R), dim3(threads), smem, stream, residual, (const float*)pending, weight, eps, (float*)out, rows, H);
    } else if (dtype == 1) {
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        st = launch_chained(add_rmsnorm_kernel<bf16>, dim3(R), dim3(threads), smem, stream, residual, (const bf16*)pending, weight, eps, (bf16*)out, rows, H);
    } else return kErrBadArgument;
    return st;
}

// ------------------------------------------------------------------ SwiGLU
// out[m,i] = silu(gu[m,i]) * gu[m,I+i],  silu(g) = g / (1 + exp(-g))
// (backends/simd/vec.go:52-59).  `gu` holds the gate columns then the up columns.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int M, int I) {
    chain_release();
    chain_wait();
    const size_t total = (size_t)M * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t m = idx / I;
        const int i = (int)(idx - m * I);
        const float g = to_f32<T>(gu[m * 2 * I + i]);
        const float u = to_f32<T>(gu[m * 2 * I + I + i]);
        const float s = g / (1.0f + expf(-g));
        out[idx] = from_f32<T>(s * u);
    }
}

GTG_API int gtg_swiglu(int dtype, const void* gu, void* out, int M, int I, cudaStream_t stream) {
    int st = 0;
    if (M <= 0 || I <= 0) return 0;
    const size_t total = (size_t)M * I;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == 0) st = launch_chained(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, M, I);
    else if (dtype == 1) st = launch_chained(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, (bf16*)out, M, I);
    else return kErrBadArgument;
    return st;
}

// ------------------------------------------------------------ rotary table
// cos_sin[n,i] = (cos, sin)(positions[n] * inv_freq[i]); the angle is a double
// product and the functions are evaluated in double, then rounded to float
// (model/llama.go:855-862).  Computed once per step for the step's tokens.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int N, int half) {
    chain_release();
    chain_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N * half) return;
    const int n = idx / half, i = idx - n * half;
    const double ang = (double)positions[n] * inv_freq[i];
    double s, c;
    sincos(ang, &s, &c);
    cos_sin[idx] = make_float2((float)c, (float)s);
}

GTG_API int gtg_rope_table(const int* positions, const double* inv_freq, float* cos_sin,
                           int N, int half, cudaStream_t stream) {
    int st = 0;
    if (N <= 0 || half <= 0) return 0;
    const int total = N * half;
    st = launch_chained(rope_table_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, positions, inv_freq, (float2*)cos_sin, N, half);
    return st;
}

// ------------------------------------------- rotation + write into the cache
// For token n with fused projections qkv[n] = [q heads | k heads | v heads]:
// rotate q in place and k on its way into the cache, a' = a*c - b*s,
// b' = a*s + b*c; copy v into the cache.  Keys are stored after rotation
// (model/llama.go:1253-1254).  Which channels (a, b) form pair i is the
// encoding's layout: half-split, (i, i + rot/2) (model/llama.go:1556-1589), or
// interleaved, (2i, 2i+1); `rot` <= hd channels of a head rotate, the rest pass
// unchanged.  cos_sin holds rot/2 (cos, sin) per token.  With n_kv_store == 0
// only the queries are rotated (a layer that reads another layer's cache).
// cos_sin == nullptr means no rotation.
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, int ld, const float2* __restrict__ cos_sin,
                                     int n_heads, int n_kv_store, int hd, int rot, int interleaved,
                                     T* __restrict__ kc, T* __restrict__ vc, long long page_stride,
                                     const int* __restrict__ block_table, int table_stride,
                                     const int* __restrict__ token_seq, const int* __restrict__ slots,
                                     const int* __restrict__ positions) {
    chain_release();
    chain_wait();
    const int n = blockIdx.x;
    const int half = hd >> 1, rhalf = rot >> 1;
    const int pos = positions[n];
    T* row = qkv + (size_t)n * ld;
    size_t cache_off = 0;
    if (n_kv_store > 0) {
        const int slot = slots[token_seq[n]];
        const int page = block_table[(size_t)slot * table_stride + pos / kPageTokens];
        cache_off = (size_t)page * page_stride + (size_t)(pos % kPageTokens) * hd;
    }
    // one item = two channels of one head: pair i of the rotated part, or two
    // consecutive channels of what passes unchanged
    const int items = (n_heads + 2 * n_kv_store) * half;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
        const int head = it / half, i = it - head * half;
        T* src = row + head * hd;
        int ia, ib;
        if (i < rhalf) { ia = interleaved ? 2 * i : i; ib = interleaved ? 2 * i + 1 : i + rhalf; }
        else { ia = rot + 2 * (i - rhalf); ib = ia + 1; }
        const float a = to_f32<T>(src[ia]), b = to_f32<T>(src[ib]);
        if (head < n_heads + n_kv_store) {
            float c = 1.f, s = 0.f;
            if (cos_sin && i < rhalf) { const float2 cs = cos_sin[(size_t)n * rhalf + i]; c = cs.x; s = cs.y; }
            const float ra = a * c - b * s, rb = a * s + b * c;
            if (head < n_heads) {
                if (i < rhalf) { src[ia] = from_f32<T>(ra); src[ib] = from_f32<T>(rb); }
            } else {
                T* dst = kc + cache_off + (size_t)(head - n_heads) * kPageTokens * hd;
                dst[ia] = i < rhalf ? from_f32<T>(ra) : src[ia];
                dst[ib] = i < rhalf ? from_f32<T>(rb) : src[ib];
            }
        } else {
            T* dst = vc + cache_off + (size_t)(head - n_heads - n_kv_store) * kPageTokens * hd;
            dst[ia] = src[ia];
            dst[ib] = src[ib];
        }
    }
}

// The same for bfloat16 with head sizes that are multiples of 16 and 16-byte
// aligned rows: one thread rotates 8 consecutive pairs with 16-byte accesses.
__global__ void rope_kv_store_bf16_vec_kernel(bf16* __restrict__ qkv, int ld, const float2* __restrict__ cos_sin,
                                              int n_heads, int n_kv_store, int hd,
                                              bf16* __restrict__ kc, bf16* __restrict__ vc, long long page_stride,
                                              const int* __restrict__ block_table, int table_stride,
                                              const int* __restrict__ token_seq, const int* __restrict__ slots,
                                              const int* __restrict__ positions) {
    chain_release();
    chain_wait();
    const int n = blockIdx.x;
    const int half = hd >> 1, chunks = half >> 3;
    const int pos = positions[n];
    bf16* row = qkv + (size_t)n * ld;
    size_t cache_off = 0;
    if (n_kv_store > 0) {
        const int slot = slots[token_seq[n]];
        const int page = block_table[(size_t)slot * table_stride + pos / kPageTokens];
        cache_off = (size_t)page * page_stride + (size_t)(pos % kPageTokens) * hd;
    }
    const int items = (n_heads + 2 * n_kv_store) * chunks;
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
        const int head = it / chunks, i = (it - head * chunks) * 8;
        bf16* src = row + head * hd;
        const uint4 av = *reinterpret_cast<const uint4*>(src + i);
        const uint4 bv = *reinterpret_cast<const uint4*>(src + i + half);
        if (head >= n_heads + n_kv_store) {                       // a value head: copy
            bf16* dst = vc + cache_off + (size_t)(head - n_heads - n_kv_store) * kPageTokens * hd;
            *reinterpret_cast<uint4*>(dst + i) = av;
            *reinterpret_cast<uint4*>(dst + i + half) = bv;
            continue;
        }
        uint4 ra = av, rb = bv;
        if (cos_sin) {
            const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)n * half + i);   // (c0,s0,c1,s1) x 4
            const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
            __nv_bfloat162* rah = reinterpret_cast<__nv_bfloat162*>(&ra);
            __nv_bfloat162* rbh = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 t = cs[j];
                const float2 a = __bfloat1622float2(ah[j]), b = __bfloat1622float2(bh[j]);
                rah[j] = __floats2bfloat162_rn(a.x * t.x - b.x * t.y, a.y * t.z - b.y * t.w);
                rbh[j] = __floats2bfloat162_rn(a.x * t.y + b.x * t.x, a.y * t.w + b.y * t.z);
            }
        }
        bf16* dst = head < n_heads ? src : kc + cache_off + (size_t)(head - n_heads) * kPageTokens * hd;
        *reinterpret_cast<uint4*>(dst + i) = ra;
        *reinterpret_cast<uint4*>(dst + i + half) = rb;
    }
}

GTG_API int gtg_rope_kv_store(int dtype, void* qkv, int ld, const float* cos_sin,
                              int n_heads, int n_kv_store, int hd, int rot, int interleaved,
                              void* kc, void* vc, long long page_stride,
                              const int* block_table, int table_stride,
                              const int* token_seq, const int* slots, const int* positions,
                              int N, cudaStream_t stream) {
    int st = 0;
    if (N <= 0) return 0;
    if (hd <= 0 || (hd & 1) || rot <= 0 || (rot & 1) || rot > hd) return kErrBadArgument;
    if (dtype == 1 && rot == hd && !interleaved && hd % 16 == 0 && ld % 8 == 0 && page_stride % 8 == 0 && ((uintptr_t)qkv % 16) == 0 &&
        ((uintptr_t)kc % 16) == 0 && ((uintptr_t)vc % 16) == 0 && ((uintptr_t)cos_sin % 16) == 0) {
        const int vec_items = (n_heads + 2 * n_kv_store) * (hd / 16);
        int t = 32;
        while (t < 256 && t < vec_items) t *= 2;
        st = launch_chained(rope_kv_store_bf16_vec_kernel, dim3(N), dim3(t), 0, stream, (bf16*)qkv, ld, (const float2*)cos_sin, n_heads, n_kv_store, hd,
            (bf16*)kc, (bf16*)vc, page_stride, block_table, table_stride, token_seq, slots, positions);
        return st;
    }
    const int items = (n_heads + 2 * n_kv_store) * (hd / 2);
    int threads = 64;
    while (threads < 512 && threads < items) threads *= 2;
    if (dtype == 0)
        st = launch_chained(rope_kv_store_kernel<float>, dim3(N), dim3(threads), 0, stream, (float*)qkv, ld, (const float2*)cos_sin, n_heads, n_kv_store, hd, rot, interleaved,
            (float*)kc, (float*)vc, page_stride, block_table, table_stride, token_seq, slots, positions);
    else if (dtype == 1)
        st = launch_chained(rope_kv_store_kernel<bf16>, dim3(N), dim3(threads), 0, stream, (bf16*)qkv, ld, (const float2*)cos_sin, n_heads, n_kv_store, hd, rot, interleaved,
            (bf16*)kc, (bf16*)vc, page_stride, block_table, table_stride, token_seq, slots, positions);
    else return kErrBadArgument;
    return st;
}

// --------------------------------------------------- advance a decode batch
// Between two decode steps that never leave the device: the sampled token
// becomes the next input, every position moves on by one and so does every
// sequence's count of generated tokens (which keys its next random draw).
__global__ void advance_kernel(int* tokens, int* positions, int* steps, const int* sampled, int B) {
    chain_wait();        // the step's metadata is written here or just before: nothing later may start early
    chain_release();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) { tokens[b] = sampled[b]; positions[b] += 1; steps[b] += 1; }
}

GTG_API int gtg_advance(int* tokens, int* positions, int* steps, const int* sampled, int B,
                        cudaStream_t stream) {
    int st = 0;
    if (B <= 0) return 0;
    st = launch_chained(advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, tokens, positions, steps, sampled, B);
    return st;
}

// ------------------------------------------- a step's cache addresses, checked
// The debug pass that stands in for a memory checker: before a kernel that finds
// its keys and values through (sequence -> slot -> block table -> page), walk the
// same indices and record the first one that would leave its array -- in a flag
// the host reads, never by trapping -- so that the host can refuse the launch.
//   mode 0  per token:    item n has sequence token_seq[n], position positions[n]
//   mode 1  per sequence: item b is read up to position positions[b] (a decode step)
//   mode 2  per sequence: item b is read up to start_pos[b] + its run in cu_seqlens (a prompt step)
// flag[0]: 0 or what is wrong (1 sequence index, 2 slot, 3 negative position or run,
// 4 position beyond the block table's row, 5 page index outside the cache);
// flag[1]: the item.
__global__ void check_cache_access_kernel(int mode, int n_items, const int* __restrict__ token_seq,
                                          const int* __restrict__ slots, const int* __restrict__ positions,
                                          const int* __restrict__ start_pos, const int* __restrict__ cu_seqlens,
                                          int n_seqs, const int* __restrict__ block_table, int table_stride,
                                          int n_slots, int n_pages, int* __restrict__ flag) {
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= n_items) return;
    int bad = 0;
    int seq = item, first_page = 0, last_pos = 0;
    if (mode == 0) {
        seq = token_seq[item];
        if (seq < 0 || seq >= n_seqs) bad = 1;
        last_pos = positions[item];
        first_page = last_pos >= 0 ? last_pos / kPageTokens : 0;          // earlier pages were other tokens' to check
    } else if (mode == 1) {
        last_pos = positions[item];
    } else {
        const int run = cu_seqlens[item + 1] - cu_seqlens[item];
        if (run < 0 || start_pos[item] < 0) bad = 3;
        last_pos = start_pos[item] + run - 1;
        if (run == 0) last_pos = -2;                                      // nothing is read
    }
    if (!bad && last_pos != -2) {
        const int slot = slots[seq];
        if (slot < 0 || slot >= n_slots) bad = 2;
        else if (last_pos < 0) bad = 3;
        else if (last_pos / kPageTokens >= table_stride) bad = 4;
        else {
            for (int p = first_page; p <= last_pos / kPageTokens; ++p) {
                const int page = block_table[(size_t)slot * table_stride + p];
                if (page < 0 || page >= n_pages) { bad = 5; break; }
            }
        }
    }
    if (bad && atomicCAS(&flag[0], 0, bad) == 0) flag[1] = item;
}

GTG_API int gtg_check_cache_access(int mode, int n_items, const int* token_seq, const int* slots,
                                   const int* positions, const int* start_pos, const int* cu_seqlens, int n_seqs,
                                   const int* block_table, int table_stride, int n_slots, int n_pages, int* flag,
                                   cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (mode < 0 || mode > 2 || flag == nullptr || slots == nullptr || block_table == nullptr) return kErrBadArgument;
    check_cache_access_kernel<<<(n_items + 127) / 128, 128, 0, stream>>>(mode, n_items, token_seq, slots, positions,
        start_pos, cu_seqlens, n_seqs, block_table, table_stride, n_slots, n_pages, flag);
    return launch_status();
}

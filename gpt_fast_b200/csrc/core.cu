// Element-wise and per-row kernels, for both precisions: token embedding,
// RMSNorm, the rotary table, rotary + cache append, length bookkeeping.
// They replace the ATen / generated kernels of gpt-fast's
// model.py:140 (embedding), :236-241 (RMSNorm), :266-293 (rotary table and
// rotation), :97-98 (cache write).  All arithmetic is 32-bit.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

// ---------------------------------------------------------------- embedding --
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int D, int V, int* status) {
    int t = blockIdx.x;
    int id = tokens[t];
    float* o = out + (size_t)t * D;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) gfb_report(status, GFB_ERR_TOKEN_RANGE, t, id);
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_to_f32(row[i]);
}

GFB_API int gfb_embed(const int* tokens, const void* table, int table_dt, float* out, int T, int D, int V,
                      int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    int threads = D >= 1024 ? 256 : 128;
    if (table_dt == GFB_BF16)
        embed_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(tokens, (const __nv_bfloat16*)table, out, D, V, status);
    else if (table_dt == GFB_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>(tokens, (const float*)table, out, D, V, status);
    else
        return gfb_fail("gfb_embed: unknown table type %d", table_dt);
    return gfb_check_launch("gfb_embed");
}

// ------------------------------------------------------------------ RMSNorm --
// out[r] = x[row(r)] * rsqrt(mean(x^2) + eps) * w, statistics and product in
// 32-bit, one rounding at the store.  `rows` (optional) gathers input rows.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int D, float eps) {
    __shared__ float scratch[32];
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    ss = gfb_block_sum(ss, scratch);
    float rstd = rsqrtf(ss / (float)D + eps);
    TO* o = out + (size_t)r * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_from_f32<TO>(xr[i] * rstd * gfb_to_f32(w[i]));
}

GFB_API int gfb_rmsnorm(const float* x, const void* w, int w_dt, void* out, int out_dt, const int* rows,
                        int R, int D, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
#define LAUNCH(TW, TO) rmsnorm_kernel<TW, TO><<<R, threads, 0, stream>>>(x, (const TW*)w, (TO*)out, rows, D, eps)
    if (w_dt == GFB_BF16 && out_dt == GFB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (w_dt == GFB_F32 && out_dt == GFB_BF16) LAUNCH(float, __nv_bfloat16);
    else if (w_dt == GFB_BF16 && out_dt == GFB_F32) LAUNCH(__nv_bfloat16, float);
    else if (w_dt == GFB_F32 && out_dt == GFB_F32) LAUNCH(float, float);
    else return gfb_fail("gfb_rmsnorm: unknown types %d %d", w_dt, out_dt);
#undef LAUNCH
    return gfb_check_launch("gfb_rmsnorm");
}

// ------------------------------------------------------------- rotary table --
// table[p][i] = (cos, sin)(p * inv_freq[i]); the angle is the 32-bit product,
// cosf/sinf are the accurate versions (this file is built without fast-math).
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ table, int P, int half) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P * half) return;
    int p = idx / half, i = idx - p * half;
    float ang = (float)p * inv_freq[i];
    table[2 * (size_t)idx] = cosf(ang);
    table[2 * (size_t)idx + 1] = sinf(ang);
}

GFB_API int gfb_rope_table(const float* inv_freq, float* table, int P, int half, cudaStream_t stream) {
    long total = (long)P * half;
    if (total <= 0) return 0;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, table, P, half);
    return gfb_check_launch("gfb_rope_table");
}

// ------------------------------------------------- rotary + cache append -----
// qkv[t] = [q heads | k heads | v heads].  q and k are rotated by the token's
// absolute position; q goes to q_out, k and v go to the token's place in the
// paged cache.  pairing 0: pairs (2i, 2i+1); pairing 1: pairs (i, i + d/2).
// append = 0: only q is produced (the layer reads a cache another layer wrote).
template <typename T>
__global__ void rope_append_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, GfbPagedKV kv, GfbBatch b,
                                   const float* __restrict__ table, int table_len, int H, int G, int d,
                                   int pairing, int append, int* status) {
    int t = blockIdx.x;
    int s = b.tok_seq[t];
    int slot = b.slots[s];
    int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    int half = d >> 1;
    bool ok = pos >= 0 && pos < table_len;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (append) {
        int pi = pos / kv.page_size, off = pos - pi * kv.page_size;
        int page = (ok && pi < kv.max_pages) ? kv.page_table[(size_t)slot * kv.max_pages + pi] : -1;
        if (page < 0 || page >= kv.n_pages) {
            ok = false;
        } else {
            size_t base = ((size_t)page * G * kv.page_size + off) * d;   // + g * page_size * d
            kdst = (T*)kv.k_pool + base;
            vdst = (T*)kv.v_pool + base;
        }
    }
    if (!ok) {
        if (threadIdx.x == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        // q_out stays defined (zeros) so that later kernels read no garbage
        for (int i = threadIdx.x; i < H * d; i += blockDim.x) q_out[(size_t)t * H * d + i] = gfb_from_f32<T>(0.f);
        return;
    }
    const T* src = qkv + (size_t)t * (H + 2 * G) * d;
    const float* cs = table + (size_t)pos * half * 2;
    int rot_pairs = (H + (append ? G : 0)) * half;
    for (int idx = threadIdx.x; idx < rot_pairs; idx += blockDim.x) {
        int head = idx / half, i = idx - head * half;
        int i0 = pairing == 0 ? 2 * i : i;
        int i1 = pairing == 0 ? 2 * i + 1 : i + half;
        const T* hsrc = src + (size_t)head * d;
        float x0 = gfb_to_f32(hsrc[i0]), x1 = gfb_to_f32(hsrc[i1]);
        float c = cs[2 * i], sn = cs[2 * i + 1];
        float o0 = x0 * c - x1 * sn;
        float o1 = x1 * c + x0 * sn;
        T* dst = head < H ? q_out + ((size_t)t * H + head) * d
                          : kdst + (size_t)(head - H) * kv.page_size * d;
        dst[i0] = gfb_from_f32<T>(o0);
        dst[i1] = gfb_from_f32<T>(o1);
    }
    if (append) {
        const T* vsrc = src + (size_t)(H + G) * d;
        for (int idx = threadIdx.x; idx < G * d; idx += blockDim.x) {
            int g = idx / d, i = idx - g * d;
            vdst[(size_t)g * kv.page_size * d + i] = vsrc[idx];
        }
    }
}

GFB_API int gfb_rope_append(const void* qkv, void* q_out, int dt,
                            void* k_pool, void* v_pool, const int* page_table, int max_pages, int page_size, int n_pages,
                            const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                            int n_seqs, int n_tokens,
                            const float* table, int table_len, int H, int G, int d, int pairing, int append,
                            int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d % 2) return gfb_fail("gfb_rope_append: head_dim %d is odd", d);
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    int work = (H + G) * d / 2;
    int threads = work >= 1024 ? 256 : 128;
    if (dt == GFB_BF16)
        rope_append_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, kv, b, table, table_len, H, G, d, pairing, append, status);
    else if (dt == GFB_F32)
        rope_append_kernel<float><<<n_tokens, threads, 0, stream>>>(
            (const float*)qkv, (float*)q_out, kv, b, table, table_len, H, G, d, pairing, append, status);
    else
        return gfb_fail("gfb_rope_append: unknown type %d", dt);
    return gfb_check_launch("gfb_rope_append");
}

// --------------------------------------------------------------- bookkeeping --
__global__ void advance_lengths_kernel(int* lengths, const int* slots, const int* cu_seqlens, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lengths[slots[i]] += cu_seqlens[i + 1] - cu_seqlens[i];
}

GFB_API int gfb_advance_lengths(int* lengths, const int* slots, const int* cu_seqlens, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    advance_lengths_kernel<<<(n + 127) / 128, 128, 0, stream>>>(lengths, slots, cu_seqlens, n);
    return gfb_check_launch("gfb_advance_lengths");
}

// out (32-bit) += y: for parts that do not fuse the residual sum into a product.
template <typename T>
__global__ void add_into_kernel(float* __restrict__ out, const T* __restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += gfb_to_f32(y[i]);
}

GFB_API int gfb_add_into(float* out, const void* y, int dt, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (dt == GFB_BF16) add_into_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(out, (const __nv_bfloat16*)y, (size_t)n);
    else if (dt == GFB_F32) add_into_kernel<float><<<blocks, 256, 0, stream>>>(out, (const float*)y, (size_t)n);
    else return gfb_fail("gfb_add_into: unknown type %d", dt);
    return gfb_check_launch("gfb_add_into");
}

// Element-wise and per-row kernels, for both precisions: token embedding,
// RMSNorm, the rotary table, rotary + cache append, length bookkeeping.
// They replace the ATen / generated kernels of gpt-fast's
// model.py:140 (embedding), :236-241 (RMSNorm), :266-293 (rotary table and
// rotation), :97-98 (cache write).  All arithmetic is 32-bit.
#include "common.cuh"

#include <cooperative_groups.h>

GFB_DEFINE_LAST_ERROR()

// ---------------------------------------------------------------- embedding --
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int D, int V, float scale, int* status) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    int t = blockIdx.x;
    int id = tokens[t];
    float* o = out + (size_t)t * D;
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) gfb_report(status, GFB_ERR_TOKEN_RANGE, t, id);
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_to_f32(row[i]) * scale;     // scale 1 changes no bit
}

// out[t] = table[tokens[t]] * scale, widened to 32-bit (scale: an architecture's factor on its embeddings; 1 for Llama).
GFB_API int gfb_embed(const int* tokens, const void* table, int table_dt, float* out, int T, int D, int V, float scale,
                      int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    int threads = D >= 1024 ? 256 : 128;
    cudaError_t e;
    if (table_dt == GFB_BF16)
        e = gfb_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, out, D, V, scale, status);
    else if (table_dt == GFB_F32)
        e = gfb_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, tokens, (const float*)table, out, D, V, scale, status);
    else
        return gfb_fail("gfb_embed: unknown table type %d", table_dt);
    return gfb_check(e, "gfb_embed");
}

// ------------------------------------------------------------------ RMSNorm --
// out[r] = x[row(r)] * rsqrt(mean(x^2) + eps) * w, statistics and product in
// 32-bit, one rounding at the store.  `rows` (optional) gathers input rows.
// With `pending` ([S][T][D] partial sums of a product split over K that still
// have to be added to the residual x) the kernel first completes the residual
// sum, x[row] += sum_s pending[s][row] in ascending s, writes x back and norms
// the result: the reduction of the split, the residual add and the norm are
// one pass over the row.
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ pending, int S, size_t slice,
                               const TW* __restrict__ w, TO* __restrict__ out, const int* __restrict__ rows,
                               int D, float eps) {
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    int r = blockIdx.x;
    size_t row = (size_t)(rows ? rows[r] : r) * D;
    float* xr = x + row;
    float ss = 0.f;
    if (pending != nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = xr[i];
            for (int k = 0; k < S; k++) v += pending[(size_t)k * slice + row + i];
            xr[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    }
    ss = gfb_block_sum(ss, scratch);
    float rstd = rsqrtf(ss / (float)D + eps);
    TO* o = out + (size_t)r * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_from_f32<TO>(xr[i] * rstd * gfb_to_f32(w[i]));
}

// The same for few rows: a cluster of NORM_CLUSTER blocks shares one row, so that a decode step's
// handful of rows keeps many SMs busy; the blocks exchange their sums of squares through
// distributed shared memory.  Needs D % (4 * NORM_CLUSTER) == 0.
constexpr int NORM_CLUSTER = 8;

template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
rmsnorm_cluster_kernel(float* __restrict__ x, const float* __restrict__ pending, int S, size_t slice,
                       const TW* __restrict__ w, TO* __restrict__ out, int D, float eps) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float scratch[32];
    __shared__ float parts[NORM_CLUSTER];                       // every block's sum of squares, pushed here by its owner
    // every block announces that it runs (its shared memory may be written from now on); the matching wait comes
    // just before the first remote write and finds the barrier complete by then
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    gfb_pdl_launch();
    const int r = blockIdx.y;
    const int chunk = D / NORM_CLUSTER;
    const int rank = (int)cluster.block_rank();
    const int c0 = rank * chunk;
    const size_t row = (size_t)r * D;
    // the usual case (chunk <= 4 * blockDim): one float4 per thread, kept in registers between the two passes
    const bool in_regs = chunk <= 4 * (int)blockDim.x;
    // the weights do not depend on the preceding kernel: they are fetched ahead of the wait for it, so that no load
    // stands between the cluster's sum and the stores
    float w4[4] = {0.f, 0.f, 0.f, 0.f};
    if (in_regs && 4 * (int)threadIdx.x < chunk) {
#pragma unroll
        for (int k = 0; k < 4; k++) w4[k] = gfb_to_f32(w[c0 + 4 * threadIdx.x + k]);
    }
    gfb_pdl_wait();
    float4 keep = make_float4(0.f, 0.f, 0.f, 0.f);
    float ss = 0.f;
    for (int i = c0 + 4 * threadIdx.x; i < c0 + chunk; i += 4 * blockDim.x) {
        float4 v = *reinterpret_cast<const float4*>(x + row + i);
        if (pending != nullptr) {
            // twelve partial sums in flight together, which covers the 8 or 9 of a decode step in one trip to L2 (the
            // last group repeats its last load instead of branching); they are added in ascending order all the same
            constexpr int W = 12;
            for (int k = 0; k < S; k += W) {
                float4 p[W];
#pragma unroll
                for (int u = 0; u < W; u++)
                    p[u] = *reinterpret_cast<const float4*>(pending + (size_t)min(k + u, S - 1) * slice + row + i);
#pragma unroll
                for (int u = 0; u < W; u++)
                    if (k + u < S) { v.x += p[u].x; v.y += p[u].y; v.z += p[u].z; v.w += p[u].w; }
            }
            *reinterpret_cast<float4*>(x + row + i) = v;
        }
        keep = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = gfb_block_sum(ss, scratch);
    // each block pushes its sum into every block's `parts`; after ONE cluster barrier all read only their own
    // shared memory, so no block has to wait for the others before it leaves
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x < NORM_CLUSTER) *cluster.map_shared_rank(&parts[rank], threadIdx.x) = ss;
    cluster.sync();
    float total = 0.f;
    for (int k = 0; k < NORM_CLUSTER; k++) total += parts[k];                                  // fixed order
    const float rstd = rsqrtf(total / (float)D + eps);
    if (in_regs) {
        const int i = c0 + 4 * threadIdx.x;
        if (i < c0 + chunk) {
            // one store of the four results (8 or 16 bytes; rows and chunks are multiples of four elements)
            struct alignas(4 * sizeof(TO)) Four { TO v[4]; } f;
            f.v[0] = gfb_from_f32<TO>(keep.x * rstd * w4[0]);
            f.v[1] = gfb_from_f32<TO>(keep.y * rstd * w4[1]);
            f.v[2] = gfb_from_f32<TO>(keep.z * rstd * w4[2]);
            f.v[3] = gfb_from_f32<TO>(keep.w * rstd * w4[3]);
            *reinterpret_cast<Four*>(out + row + i) = f;
        }
        return;
    }
    for (int i = c0 + 4 * threadIdx.x; i < c0 + chunk; i += 4 * blockDim.x) {
        const float4 v = *reinterpret_cast<const float4*>(x + row + i);
        TO* o = out + row + i;
        o[0] = gfb_from_f32<TO>(v.x * rstd * gfb_to_f32(w[i]));
        o[1] = gfb_from_f32<TO>(v.y * rstd * gfb_to_f32(w[i + 1]));
        o[2] = gfb_from_f32<TO>(v.z * rstd * gfb_to_f32(w[i + 2]));
        o[3] = gfb_from_f32<TO>(v.w * rstd * gfb_to_f32(w[i + 3]));
    }
}

// One block per row with the row held in registers: a single pass over x (float4 loads),
// packed stores.  For D % 4 == 0 and D <= 4 * VEC_MAX * blockDim.
constexpr int NORM_VEC_MAX = 8;

template <typename TW, typename TO>
__global__ void rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ pending, int S, size_t slice,
                                   const TW* __restrict__ w, TO* __restrict__ out, const int* __restrict__ rows, int D, float eps) {
    __shared__ float scratch[32];
    gfb_pdl_launch();
    const int r = blockIdx.x;
    const int nvec = D >> 2;
    // the weights do not depend on the preceding kernel: fetched ahead of the wait for it, so that no load stands
    // between the row's sum and the stores
    float wk[NORM_VEC_MAX][4];
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; k++) {
        int i = threadIdx.x + k * blockDim.x;
#pragma unroll
        for (int e = 0; e < 4; e++) wk[k][e] = i < nvec ? gfb_to_f32(w[4 * i + e]) : 0.f;
    }
    gfb_pdl_wait();
    const size_t row = (size_t)(rows ? rows[r] : r) * D;
    float4* xr = reinterpret_cast<float4*>(x + row);
    float4 v[NORM_VEC_MAX];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; k++) {
        int i = threadIdx.x + k * blockDim.x;
        v[k] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (pending != nullptr) {
        // the row's pending partial sums, one after the other (ascending), each with all of a thread's loads in flight
        for (int p = 0; p < S; p++) {
            const float4* pr = reinterpret_cast<const float4*>(pending + (size_t)p * slice + row);
            float4 a[NORM_VEC_MAX];
#pragma unroll
            for (int k = 0; k < NORM_VEC_MAX; k++) {
                int i = threadIdx.x + k * blockDim.x;
                a[k] = i < nvec ? pr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < NORM_VEC_MAX; k++) { v[k].x += a[k].x; v[k].y += a[k].y; v[k].z += a[k].z; v[k].w += a[k].w; }
        }
#pragma unroll
        for (int k = 0; k < NORM_VEC_MAX; k++) {
            int i = threadIdx.x + k * blockDim.x;
            if (i < nvec) xr[i] = v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; k++) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = gfb_block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int k = 0; k < NORM_VEC_MAX; k++) {
        int i = threadIdx.x + k * blockDim.x;
        if (i < nvec) {
            float o0 = v[k].x * rstd * wk[k][0], o1 = v[k].y * rstd * wk[k][1];
            float o2 = v[k].z * rstd * wk[k][2], o3 = v[k].w * rstd * wk[k][3];
            TO* o = out + (size_t)r * D + 4 * i;
            if (sizeof(TO) == 4) {
                *reinterpret_cast<float4*>(o) = make_float4(o0, o1, o2, o3);
            } else {
                __nv_bfloat162 a = __floats2bfloat162_rn(o0, o1), b = __floats2bfloat162_rn(o2, o3);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&a);
                pk.y = *reinterpret_cast<uint32_t*>(&b);
                *reinterpret_cast<uint2*>(o) = pk;
            }
        }
    }
}

GFB_API int gfb_rmsnorm(float* x, const float* pending, int S, long slice, const void* w, int w_dt, void* out, int out_dt,
                        const int* rows, int R, int D, float eps, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (pending != nullptr && rows != nullptr) return gfb_fail("gfb_rmsnorm: pending partial sums cannot be combined with a row gather");
    cudaError_t e;
    if (rows == nullptr && R <= 128 && D >= 1024 && D % (4 * NORM_CLUSTER) == 0) {
        dim3 grid(NORM_CLUSTER, R);
#define CLAUNCH(TW, TO) e = gfb_launch_cluster(rmsnorm_cluster_kernel<TW, TO>, grid, dim3(128), 0, stream, NORM_CLUSTER, x, pending, S, (size_t)slice, (const TW*)w, (TO*)out, D, eps)
        if (w_dt == GFB_BF16 && out_dt == GFB_BF16) CLAUNCH(__nv_bfloat16, __nv_bfloat16);
        else if (w_dt == GFB_F32 && out_dt == GFB_BF16) CLAUNCH(float, __nv_bfloat16);
        else if (w_dt == GFB_BF16 && out_dt == GFB_F32) CLAUNCH(__nv_bfloat16, float);
        else if (w_dt == GFB_F32 && out_dt == GFB_F32) CLAUNCH(float, float);
        else return gfb_fail("gfb_rmsnorm: unknown types %d %d", w_dt, out_dt);
#undef CLAUNCH
        return gfb_check(e, "gfb_rmsnorm (cluster)");
    }
    int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    if ((pending == nullptr || slice % 4 == 0) && D % 4 == 0 && D <= 4 * NORM_VEC_MAX * threads) {
        // few threads with many loads each: more rows are resident per SM and every thread has 8 loads in flight
        int vthreads = ((D / 4 + NORM_VEC_MAX - 1) / NORM_VEC_MAX + 31) / 32 * 32;
        if (vthreads < 64) vthreads = 64;
#define VLAUNCH(TW, TO) e = gfb_launch(rmsnorm_vec_kernel<TW, TO>, dim3(R), dim3(vthreads), 0, stream, x, pending, S, (size_t)slice, (const TW*)w, (TO*)out, rows, D, eps)
        if (w_dt == GFB_BF16 && out_dt == GFB_BF16) VLAUNCH(__nv_bfloat16, __nv_bfloat16);
        else if (w_dt == GFB_F32 && out_dt == GFB_BF16) VLAUNCH(float, __nv_bfloat16);
        else if (w_dt == GFB_BF16 && out_dt == GFB_F32) VLAUNCH(__nv_bfloat16, float);
        else if (w_dt == GFB_F32 && out_dt == GFB_F32) VLAUNCH(float, float);
        else return gfb_fail("gfb_rmsnorm: unknown types %d %d", w_dt, out_dt);
#undef VLAUNCH
        return gfb_check(e, "gfb_rmsnorm (vector)");
    }
#define LAUNCH(TW, TO) e = gfb_launch(rmsnorm_kernel<TW, TO>, dim3(R), dim3(threads), 0, stream, x, pending, S, (size_t)slice, (const TW*)w, (TO*)out, rows, D, eps)
    if (w_dt == GFB_BF16 && out_dt == GFB_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (w_dt == GFB_F32 && out_dt == GFB_BF16) LAUNCH(float, __nv_bfloat16);
    else if (w_dt == GFB_BF16 && out_dt == GFB_F32) LAUNCH(__nv_bfloat16, float);
    else if (w_dt == GFB_F32 && out_dt == GFB_F32) LAUNCH(float, float);
    else return gfb_fail("gfb_rmsnorm: unknown types %d %d", w_dt, out_dt);
#undef LAUNCH
    return gfb_check(e, "gfb_rmsnorm");
}

// x += sum_s pending[s] (ascending s): completes a residual sum whose product was split over K.
__global__ void add_partials_kernel(float* __restrict__ x, const float* __restrict__ pending, int S, size_t n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    for (int k = 0; k < S; k++) v += pending[(size_t)k * n + i];
    x[i] = v;
}

GFB_API int gfb_add_partials(float* x, const float* pending, int S, long n, cudaStream_t stream) {
    if (n <= 0 || S <= 0) return 0;
    cudaError_t e = gfb_launch(add_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, pending, S, (size_t)n);
    return gfb_check(e, "gfb_add_partials");
}

// ------------------------------------------------------------- rotary table --
// table[p][i] = (cos, sin)(p * inv_freq[i]); the angle is the 32-bit product,
// cosf/sinf are the accurate versions (this file is built without fast-math).
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ table, int P, int half) {
    gfb_pdl_launch();
    gfb_pdl_wait();
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
    cudaError_t e = gfb_launch(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, inv_freq, table, P, half);
    return gfb_check(e, "gfb_rope_table");
}

// ------------------------------------------------- rotary + cache append -----
// qkv[t] = [q heads | k heads | v heads].  q and k are rotated by the token's
// absolute position; q goes to q_out, k and v go to the token's place in the
// paged cache.  pairing 0: pairs (2i, 2i+1); pairing 1: pairs (i, i + d/2).
// append = 0: only q is produced (the layer reads a cache another layer wrote).
// The input is either qkv in the model's type, or (PARTIAL) the 32-bit partial
// sums [S][T][(H+2G)d] of a product split over K, which are summed here in
// ascending s: the split's reduction costs no kernel of its own.
// One thread per pair of elements: block y of token x handles 256 pairs.
template <typename T, bool PARTIAL>
__global__ void rope_append_kernel(const void* __restrict__ src_any, int S, size_t slice, T* __restrict__ q_out,
                                   GfbPagedKV kv, GfbBatch b, const float* __restrict__ table, int table_len,
                                   int H, int G, int d, int pairing, int append, int* status) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x;
    const int half = d >> 1;
    const int n_rot = (H + (append ? G : 0)) * half;          // rotated pairs
    const int n_items = n_rot + (append ? G * half : 0);      // + pairs of v that are copied
    const int item = blockIdx.y * blockDim.x + threadIdx.x;
    if (item >= n_items) return;
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    const int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    bool ok = pos >= 0 && pos < table_len;
    size_t cache_base = 0;
    if (append) {
        int pi = pos / kv.page_size, off = pos - pi * kv.page_size;
        int page = (ok && pi < kv.max_pages) ? kv.page_table[(size_t)slot * kv.max_pages + pi] : -1;
        if (page < 0 || page >= kv.n_pages) ok = false;
        else cache_base = ((size_t)page * G * kv.page_size + off) * d;          // + g * page_size * d
    }
    const bool rot = item < n_rot;
    const int head = rot ? item / half : H + G + (item - n_rot) / half;
    const int i = rot ? item - head * half : (item - n_rot) % half;
    const int i0 = (rot && pairing == 1) ? i : 2 * i;
    const int i1 = (rot && pairing == 1) ? i + half : 2 * i + 1;
    if (!ok) {
        if (item == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        if (head < H) {                                       // q stays defined so that later kernels read no garbage
            T* dst = q_out + ((size_t)t * H + head) * d;
            dst[i0] = gfb_from_f32<T>(0.f);
            dst[i1] = gfb_from_f32<T>(0.f);
        }
        return;
    }
    const size_t W = (size_t)(H + 2 * G) * d;
    const size_t e0 = (size_t)t * W + (size_t)head * d + i0, e1 = (size_t)t * W + (size_t)head * d + i1;
    float x0, x1;
    if (PARTIAL) {
        const float* p = (const float*)src_any;
        x0 = 0.f; x1 = 0.f;
        for (int k = 0; k < S; k++) { x0 += p[(size_t)k * slice + e0]; x1 += p[(size_t)k * slice + e1]; }
    } else {
        const T* p = (const T*)src_any;
        x0 = gfb_to_f32(p[e0]); x1 = gfb_to_f32(p[e1]);
    }
    T* dst;
    if (head < H) dst = q_out + ((size_t)t * H + head) * d;
    else if (head < H + G) dst = (T*)kv.k_pool + cache_base + (size_t)(head - H) * kv.page_size * d;
    else dst = (T*)kv.v_pool + cache_base + (size_t)(head - H - G) * kv.page_size * d;
    if (rot) {
        const float* cs = table + ((size_t)pos * half + i) * 2;
        float c = cs[0], sn = cs[1];
        dst[i0] = gfb_from_f32<T>(x0 * c - x1 * sn);
        dst[i1] = gfb_from_f32<T>(x1 * c + x0 * sn);
    } else {
        dst[i0] = gfb_from_f32<T>(x0);
        dst[i1] = gfb_from_f32<T>(x1);
    }
}

// Fast path for many tokens: bfloat16 qkv, interleaved pairs, head_dim % 8 == 0.  One thread moves
// 8 elements (4 pairs): a 16-byte load of qkv, two 16-byte loads of (cos, sin), a 16-byte store.
constexpr int ROPE_VEC_ITEMS = 4;

__global__ void __launch_bounds__(256)
rope_append_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                       GfbPagedKV kv, GfbBatch b, const float* __restrict__ table, int table_len,
                       int H, int G, int d, int append, int* status) {
    gfb_pdl_launch();
    // one block per token: the chain token -> sequence -> slot -> position -> page is walked once per block, and a
    // thread's items (8 elements each, up to ROPE_VEC_ITEMS of them) are loaded together.  The first links of the
    // chain are the host's bookkeeping of this step and are read ahead of the wait for the preceding kernel; the
    // lengths are advanced by a kernel (the last one of the previous step) and are read behind it.
    const int t = blockIdx.x;
    const int d8 = d >> 3;
    const int n_items = (H + (append ? 2 * G : 0)) * d8;
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    const int q_off = t - b.cu_seqlens[s];
    gfb_pdl_wait();
    const int pos = b.lengths[slot] + q_off;
    bool ok = pos >= 0 && pos < table_len;
    size_t cache_base = 0;
    if (append) {
        int pi = pos / kv.page_size, off = pos - pi * kv.page_size;
        int page = (ok && pi < kv.max_pages) ? kv.page_table[(size_t)slot * kv.max_pages + pi] : -1;
        if (page < 0 || page >= kv.n_pages) ok = false;
        else cache_base = ((size_t)page * G * kv.page_size + off) * d;
    }
    if (!ok) {
        if (threadIdx.x == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        for (int item = threadIdx.x; item < H * d8; item += blockDim.x)
            *reinterpret_cast<uint4*>(q_out + (size_t)t * H * d + (size_t)item * 8) = make_uint4(0, 0, 0, 0);
        return;
    }
    const __nv_bfloat16* src = qkv + (size_t)t * (H + 2 * G) * d;
    const float* cs_row = table + (size_t)pos * (d >> 1) * 2;
    for (int base = 0; base < n_items; base += ROPE_VEC_ITEMS * blockDim.x) {
        uint4 raw[ROPE_VEC_ITEMS];
        float4 cs0[ROPE_VEC_ITEMS], cs1[ROPE_VEC_ITEMS];
#pragma unroll
        for (int u = 0; u < ROPE_VEC_ITEMS; u++) {
            const int item = base + u * blockDim.x + threadIdx.x;
            if (item < n_items) {
                raw[u] = *reinterpret_cast<const uint4*>(src + (size_t)item * 8);       // items lie one after the other in qkv
                const int c = item % d8;
                const float4* cs = reinterpret_cast<const float4*>(cs_row + c * 8);
                cs0[u] = cs[0];                                  // (cos, sin) of pairs 0,1 and 2,3
                cs1[u] = cs[1];
            }
        }
#pragma unroll
        for (int u = 0; u < ROPE_VEC_ITEMS; u++) {
            const int item = base + u * blockDim.x + threadIdx.x;
            if (item >= n_items) continue;
            const int head = item / d8, c = item - head * d8;    // head over q, k, v; c: which 8 elements
            __nv_bfloat16* dst;
            if (head < H) dst = q_out + ((size_t)t * H + head) * d;
            else if (head < H + G) dst = (__nv_bfloat16*)kv.k_pool + cache_base + (size_t)(head - H) * kv.page_size * d;
            else dst = (__nv_bfloat16*)kv.v_pool + cache_base + (size_t)(head - H - G) * kv.page_size * d;
            if (head < H + G) {
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&raw[u]);
                float2 x0 = __bfloat1622float2(p2[0]), x1 = __bfloat1622float2(p2[1]);
                float2 x2 = __bfloat1622float2(p2[2]), x3 = __bfloat1622float2(p2[3]);
                p2[0] = __floats2bfloat162_rn(x0.x * cs0[u].x - x0.y * cs0[u].y, x0.y * cs0[u].x + x0.x * cs0[u].y);
                p2[1] = __floats2bfloat162_rn(x1.x * cs0[u].z - x1.y * cs0[u].w, x1.y * cs0[u].z + x1.x * cs0[u].w);
                p2[2] = __floats2bfloat162_rn(x2.x * cs1[u].x - x2.y * cs1[u].y, x2.y * cs1[u].x + x2.x * cs1[u].y);
                p2[3] = __floats2bfloat162_rn(x3.x * cs1[u].z - x3.y * cs1[u].w, x3.y * cs1[u].z + x3.x * cs1[u].w);
            }
            *reinterpret_cast<uint4*>(dst + c * 8) = raw[u];
        }
    }
}

// src: qkv [T, (H+2G)d] of type dt, or, with n_partials > 0, float partial sums [n_partials][T][(H+2G)d].
GFB_API int gfb_rope_append(const void* src, int n_partials, void* q_out, int dt,
                            void* k_pool, void* v_pool, const int* page_table, int max_pages, int page_size, int n_pages,
                            const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                            int n_seqs, int n_tokens,
                            const float* table, int table_len, int H, int G, int d, int pairing, int append,
                            int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d % 2) return gfb_fail("gfb_rope_append: head_dim %d is odd", d);
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    if (dt == GFB_BF16 && n_partials == 0 && pairing == 0 && d % 8 == 0 && n_tokens >= 64) {
        int vitems = (H + (append ? 2 * G : 0)) * (d / 8);
        dim3 vgrid(n_tokens);
        int vthreads = ((vitems + ROPE_VEC_ITEMS - 1) / ROPE_VEC_ITEMS + 31) / 32 * 32;
        if (vthreads > 256) vthreads = 256;
        cudaError_t ve = gfb_launch(rope_append_vec_kernel, vgrid, dim3(vthreads), 0, stream, (const __nv_bfloat16*)src,
                                    (__nv_bfloat16*)q_out, kv, b, table, table_len, H, G, d, append, status);
        return gfb_check(ve, "gfb_rope_append (vector)");
    }
    int items = (H + (append ? 2 * G : 0)) * (d / 2);
    dim3 grid(n_tokens, (items + 255) / 256);
    if (grid.y > 65535) return gfb_fail("gfb_rope_append: %d heads of %d exceed the grid", H + 2 * G, d);
    size_t slice = (size_t)n_tokens * (H + 2 * G) * d;
    cudaError_t e;
#define GO(T, P) e = gfb_launch(rope_append_kernel<T, P>, grid, dim3(256), 0, stream, src, n_partials, slice, (T*)q_out, kv, b, table, table_len, H, G, d, pairing, append, status)
    if (dt == GFB_BF16 && n_partials > 0) GO(__nv_bfloat16, true);
    else if (dt == GFB_BF16) GO(__nv_bfloat16, false);
    else if (dt == GFB_F32 && n_partials > 0) GO(float, true);
    else if (dt == GFB_F32) GO(float, false);
    else return gfb_fail("gfb_rope_append: unknown type %d", dt);
#undef GO
    return gfb_check(e, "gfb_rope_append");
}

// --------------------------------------------------------------- bookkeeping --
__global__ void advance_lengths_kernel(int* lengths, const int* slots, const int* cu_seqlens, int n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) lengths[slots[i]] += cu_seqlens[i + 1] - cu_seqlens[i];
}

GFB_API int gfb_advance_lengths(int* lengths, const int* slots, const int* cu_seqlens, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    cudaError_t e = gfb_launch(advance_lengths_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, lengths, slots, cu_seqlens, n);
    return gfb_check(e, "gfb_advance_lengths");
}

// out (32-bit) += y: for parts that do not fuse the residual sum into a product.
template <typename T>
__global__ void add_into_kernel(float* __restrict__ out, const T* __restrict__ y, size_t n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += gfb_to_f32(y[i]);
}

GFB_API int gfb_add_into(float* out, const void* y, int dt, long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e;
    if (dt == GFB_BF16) e = gfb_launch(add_into_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, out, (const __nv_bfloat16*)y, (size_t)n);
    else if (dt == GFB_F32) e = gfb_launch(add_into_kernel<float>, dim3(blocks), dim3(256), 0, stream, out, (const float*)y, (size_t)n);
    else return gfb_fail("gfb_add_into: unknown type %d", dt);
    return gfb_check(e, "gfb_add_into");
}

// x = cap * tanh(x / cap), in 32-bit, in place: a soft cap on logits (an architecture's option; Llama has none).
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

GFB_API int gfb_softcap(float* x, long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return gfb_fail("gfb_softcap: the cap must be positive, got %g", (double)cap);
    cudaError_t e = gfb_launch(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, (size_t)n, cap);
    return gfb_check(e, "gfb_softcap");
}

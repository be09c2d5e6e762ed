// Causal grouped-query attention over the paged cache, for any head size, any
// number of heads and groups, any mix of query lengths, both precisions.
//
// It stands where gpt-fast expands K/V to all heads and calls SDPA over the
// whole cache with a boolean mask (model.py:209-211): query head h reads
// key/value head h / (H/G); the key at position j is visible to the query at
// position p iff j <= p (and p - j < window when a window is set); scores are
// scaled by `scale`; softmax is 32-bit.
//
// One block per (token, query head).  Keys are visited in chunks of 128 that
// start at multiples of 128 of the ABSOLUTE position, with an online softmax
// between chunks, so a query's result is the same bits whether its token came
// in a long prompt, alone, or in any batch.  This is the kernel of the 32-bit
// path and the fallback of the bfloat16 path; the fast bfloat16 kernels live
// in files of their own.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

constexpr int CHUNK = 128;      // keys per step = threads per block
constexpr int MAX_DPT = 4;      // head_dim <= CHUNK * MAX_DPT

template <typename T>
__global__ void __launch_bounds__(CHUNK)
attention_generic_kernel(const T* __restrict__ q, T* __restrict__ out, GfbPagedKV kv, GfbBatch b,
                         int H, int G, int d, float scale, int window, int* status) {
    extern __shared__ float smem[];
    float* qs = smem;              // [d]
    float* ps = smem + d;          // [CHUNK]
    __shared__ float scratch[32];
    __shared__ int page_of[CHUNK]; // page ids of the current chunk (2 pages of 64, or fewer larger ones)
    gfb_pdl_launch();
    gfb_pdl_wait();

    int t = blockIdx.x, h = blockIdx.y;
    int g = h / (H / G);
    int s = b.tok_seq[t];
    int slot = b.slots[s];
    int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    const T* qrow = q + ((size_t)t * H + h) * d;
    for (int i = threadIdx.x; i < d; i += CHUNK) qs[i] = gfb_to_f32(qrow[i]) * scale;

    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const int* pt = kv.page_table + (size_t)slot * kv.max_pages;
    const size_t head_off = (size_t)g * kv.page_size * d;
    const size_t page_stride = (size_t)G * kv.page_size * d;

    float m_run = -INFINITY, l_run = 0.f;
    float acc[MAX_DPT];
#pragma unroll
    for (int i = 0; i < MAX_DPT; i++) acc[i] = 0.f;

    for (int c0 = (lo / CHUNK) * CHUNK; c0 <= pos; c0 += CHUNK) {
        __syncthreads();           // qs ready (first pass); ps / page_of free (later passes)
        int j = c0 + threadIdx.x;
        bool live = j >= lo && j <= pos;
        int page = -1;
        if (live) {
            int pi = j / kv.page_size;
            page = pi < kv.max_pages ? pt[pi] : -1;
            if (page < 0 || page >= kv.n_pages) {
                gfb_report(status, GFB_ERR_PAGE_TABLE, slot, pi);
                live = false;
                page = -1;
            }
        }
        page_of[threadIdx.x] = page;
        float sc = -INFINITY;
        if (live) {
            const T* krow = (const T*)kv.k_pool + (size_t)page * page_stride + head_off
                            + (size_t)(j % kv.page_size) * d;
            float dot = 0.f;
            for (int i = 0; i < d; i++) dot = fmaf(qs[i], gfb_to_f32(krow[i]), dot);
            sc = dot;
        }
        float m_new = fmaxf(m_run, gfb_block_max(sc, scratch));
        float p = live ? expf(sc - m_new) : 0.f;
        ps[threadIdx.x] = p;
        float l_chunk = gfb_block_sum(p, scratch);     // also orders the ps / page_of stores
        float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        l_run = l_run * corr + l_chunk;
        m_run = m_new;
        int nkeys = min(CHUNK, pos - c0 + 1);
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = threadIdx.x + r * CHUNK;
            if (dim < d) {
                float a = acc[r] * corr;
                for (int jj = 0; jj < nkeys; jj++) {
                    int pg = page_of[jj];
                    if (pg < 0) continue;
                    const T* vrow = (const T*)kv.v_pool + (size_t)pg * page_stride + head_off
                                    + (size_t)((c0 + jj) % kv.page_size) * d;
                    a = fmaf(ps[jj], gfb_to_f32(vrow[dim]), a);
                }
                acc[r] = a;
            }
        }
    }
    float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* orow = out + ((size_t)t * H + h) * d;
#pragma unroll
    for (int r = 0; r < MAX_DPT; r++) {
        int dim = threadIdx.x + r * CHUNK;
        if (dim < d) orow[dim] = gfb_from_f32<T>(acc[r] * inv);
    }
}

GFB_API int gfb_attention_generic(const void* q, void* out, int dt,
                                  void* k_pool, void* v_pool, const int* page_table, int max_pages, int page_size,
                                  int n_pages,
                                  const int* cu_seqlens, const int* tok_seq, const int* slots, const int* lengths,
                                  int n_seqs, int n_tokens, int H, int G, int d, float scale, int window,
                                  int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (d > CHUNK * MAX_DPT) return gfb_fail("gfb_attention_generic: head_dim %d exceeds %d", d, CHUNK * MAX_DPT);
    if (G <= 0 || H % G) return gfb_fail("gfb_attention_generic: %d heads do not divide into %d groups", H, G);
    if (H > 65535) return gfb_fail("gfb_attention_generic: %d heads exceed the grid limit", H);
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    dim3 grid(n_tokens, H);
    size_t smem = (size_t)(d + CHUNK) * sizeof(float);
    cudaError_t e;
    if (dt == GFB_BF16)
        e = gfb_launch(attention_generic_kernel<__nv_bfloat16>, grid, dim3(CHUNK), smem, stream,
                       (const __nv_bfloat16*)q, (__nv_bfloat16*)out, kv, b, H, G, d, scale, window, status);
    else if (dt == GFB_F32)
        e = gfb_launch(attention_generic_kernel<float>, grid, dim3(CHUNK), smem, stream,
                       (const float*)q, (float*)out, kv, b, H, G, d, scale, window, status);
    else
        return gfb_fail("gfb_attention_generic: unknown type %d", dt);
    return gfb_check(e, "gfb_attention_generic");
}

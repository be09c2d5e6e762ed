// bfloat16 attention kernels of the serving path (the 32-bit path and odd
// sizes use attention_generic.cu).  They stand where gpt-fast expands K/V to all
// heads and calls SDPA over the whole cache (model.py:209-211).
//
// attn_decode: one new token per sequence.  A block owns (sequence, key/value
// head, slice of the sequence's pages) and serves all query heads of the group
// from one pass over the keys and values, so each cached byte is read once per
// group, not once per head.  Pages (64 tokens x head_dim, contiguous per head)
// are brought to shared memory several pages ahead (cp.async; TMA in the
// tensor-core version).  Scores,
// softmax and the weighted sum are 32-bit.  With more than one slice per
// sequence the blocks write (max, sum, unnormalised output) to scratch and
// attn_combine merges the slices in ascending order.
#include <cuda.h>

#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

namespace {

constexpr int PAGE = 64;
constexpr int THREADS = 128;
constexpr int MAX_REP = 8;          // query heads per key/value head
constexpr int MAX_DPT = 2;          // head_dim <= THREADS * MAX_DPT
// K/V tile pairs of the tensor-core decode kernel: NBUF - 1 pages are in flight per block.  3 lets two blocks share
// an SM and 2 three; 5 (one block per SM) is for the smallest grids, where a short context is then requested all at once.
constexpr int DECODE_NBUF_MANY = 3, DECODE_NBUF_FEW = 5, DECODE_NBUF_SHORT = 2;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
// A decode step reads every cached key and value once, so their lines are marked to be evicted first and leave L2
// to what is read again within the step.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// A box of a page ([64 tokens][64 dims], 128-byte swizzle) by TMA; its bytes are counted on a shared-memory barrier.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
}
constexpr unsigned long long PAGE_WAIT_LIMIT_NS = 1000000000ull;   // a page that has not come after a second is given up
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// q: [T, H, d]; out: [T, H*d]; scratch_o: [T, H, S, d] f32; scratch_ml: [T, H, S, 2] f32
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ scratch_o, float* __restrict__ scratch_ml,
                   GfbPagedKV kv, GfbBatch b, int H, int G, int d, float scale_log2e, int window, int splits, int* status) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int rep = H / G;
    const int tile_bytes = PAGE * d * 2;
    __nv_bfloat16* kbuf[2] = {(__nv_bfloat16*)smem, (__nv_bfloat16*)(smem + 2 * tile_bytes)};
    __nv_bfloat16* vbuf[2] = {(__nv_bfloat16*)(smem + tile_bytes), (__nv_bfloat16*)(smem + 3 * tile_bytes)};
    float* qs = (float*)(smem + 4 * tile_bytes);          // [rep][d], pre-scaled
    float* ps = qs + rep * d;                             // [rep][PAGE]
    __shared__ float red[MAX_REP][2];      // per head: (rescale of what was summed so far, sum of this tile)
    __shared__ float mrun[MAX_REP];        // per head: running maximum

    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x, g = blockIdx.y, z = blockIdx.z;
    const int s = b.tok_seq[t];
    const int slot = b.slots[s];
    const int pos = b.lengths[slot] + (t - b.cu_seqlens[s]);
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first_page = lo / PAGE, last_page = pos / PAGE;
    const int n_pages = last_page - first_page + 1;
    const int per = (n_pages + splits - 1) / splits;
    const int p0 = first_page + z * per;
    const int p1 = min(last_page + 1, p0 + per);
    const int tid = threadIdx.x;

    for (int i = tid; i < rep * d; i += THREADS) {
        int h = i / d;
        qs[i] = __bfloat162float(q[((size_t)t * H + g * rep + h) * d + (i - h * d)]) * scale_log2e;
    }

    if (tid < MAX_REP) mrun[tid] = -INFINITY;
    float l_run[MAX_REP], acc[MAX_REP][MAX_DPT];
#pragma unroll
    for (int h = 0; h < MAX_REP; h++) {
        l_run[h] = 0.f;
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) acc[h][r] = 0.f;
    }

    const int* pt = kv.page_table + (size_t)slot * kv.max_pages;
    const int chunks = tile_bytes / 16;                   // 16-byte pieces of one tile
    auto issue = [&](int page_index, int buf) {
        int page = pt[page_index];
        if (page < 0 || page >= kv.n_pages) {
            if (tid == 0) gfb_report(status, GFB_ERR_PAGE_TABLE, slot, page_index);
            page = 0;                                     // read a valid page; its scores are masked below
        }
        const uint8_t* ksrc = (const uint8_t*)kv.k_pool + ((size_t)page * G + g) * tile_bytes;
        const uint8_t* vsrc = (const uint8_t*)kv.v_pool + ((size_t)page * G + g) * tile_bytes;
        for (int c = tid; c < chunks; c += THREADS) {
            cp_async16((uint8_t*)kbuf[buf] + c * 16, ksrc + c * 16);
            cp_async16((uint8_t*)vbuf[buf] + c * 16, vsrc + c * 16);
        }
    };

    if (p0 < p1) issue(p0, 0);
    cp_async_commit();
    const int key = tid & (PAGE - 1), hg = tid >> 6;      // QK: 64 keys x 2 head groups
    const int d8 = d >> 3;
    for (int p = p0; p < p1; p++) {
        const int buf = (p - p0) & 1;
        if (p + 1 < p1) issue(p + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                  // tile p landed; qs ready (first pass)

        // scores of this thread's key for heads hg, hg+2, ...
        const int j = p * PAGE + key;
        const bool live = j >= lo && j <= pos;
        float dot[MAX_REP / 2];
#pragma unroll
        for (int i = 0; i < MAX_REP / 2; i++) dot[i] = 0.f;
        const uint4* krow = reinterpret_cast<const uint4*>(kbuf[buf] + (size_t)key * d);
        const int start = key % d8;                       // rotate the start: neighbouring keys hit different banks
        for (int c = 0; c < d8; c++) {
            int cc = start + c;
            if (cc >= d8) cc -= d8;
            uint4 raw = krow[cc];
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float kf[8];
#pragma unroll
            for (int e = 0; e < 4; e++) { float2 f = __bfloat1622float2(k2[e]); kf[2 * e] = f.x; kf[2 * e + 1] = f.y; }
#pragma unroll
            for (int i = 0; i < MAX_REP / 2; i++) {
                int h = hg + 2 * i;
                if (h < rep) {
                    const float4* qv = reinterpret_cast<const float4*>(qs + h * d + cc * 8);
                    float4 a = qv[0], c4 = qv[1];
                    dot[i] += a.x * kf[0] + a.y * kf[1] + a.z * kf[2] + a.w * kf[3]
                            + c4.x * kf[4] + c4.y * kf[5] + c4.z * kf[6] + c4.w * kf[7];
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_REP / 2; i++) {
            int h = hg + 2 * i;
            if (h < rep) ps[h * PAGE + key] = live ? dot[i] : -INFINITY;
        }
        __syncthreads();

        // per head: tile max and probabilities (warp w serves heads w, w+4)
        const int warp = tid >> 5, lane = tid & 31;
        for (int h = warp; h < rep; h += THREADS / 32) {
            float s0 = ps[h * PAGE + lane], s1 = ps[h * PAGE + 32 + lane];
            float mx = gfb_warp_max(fmaxf(s0, s1));
            float m_old = mrun[h];
            float m_new = fmaxf(m_old, mx);
            float e0 = (s0 == -INFINITY) ? 0.f : exp2f(s0 - m_new);
            float e1 = (s1 == -INFINITY) ? 0.f : exp2f(s1 - m_new);
            ps[h * PAGE + lane] = e0;
            ps[h * PAGE + 32 + lane] = e1;
            float sum = gfb_warp_sum(e0 + e1);
            if (lane == 0) {
                red[h][0] = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_new);
                red[h][1] = sum;
                mrun[h] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < MAX_REP; h++) {
            if (h < rep) {
                float corr = red[h][0];
                l_run[h] = l_run[h] * corr + red[h][1];
#pragma unroll
                for (int r = 0; r < MAX_DPT; r++) acc[h][r] *= corr;
            }
        }
        // weighted sum: thread owns dims tid, tid + 128
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = tid + r * THREADS;
            if (dim < d) {
                const __nv_bfloat16* vcol = vbuf[buf] + dim;
                for (int jj = 0; jj < PAGE; jj++) {
                    float v = __bfloat162float(vcol[(size_t)jj * d]);
#pragma unroll
                    for (int h = 0; h < MAX_REP; h++)
                        if (h < rep) acc[h][r] = fmaf(ps[h * PAGE + jj], v, acc[h][r]);
                }
            }
        }
        __syncthreads();                                  // ps and this buffer are reused next round
    }
    cp_async_wait<0>();
    __syncthreads();                                      // mrun is final (also when this block had no page)

#pragma unroll
    for (int h = 0; h < MAX_REP; h++) {
        if (h >= rep) continue;
        const int head = g * rep + h;
#pragma unroll
        for (int r = 0; r < MAX_DPT; r++) {
            int dim = tid + r * THREADS;
            if (dim >= d) continue;
            if (splits == 1) {
                float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
                out[((size_t)t * H + head) * d + dim] = __float2bfloat16_rn(acc[h][r] * inv);
            } else {
                scratch_o[(((size_t)t * H + head) * splits + z) * d + dim] = acc[h][r];
            }
        }
        if (splits > 1 && tid == 0) {
            float* ml = scratch_ml + (((size_t)t * H + head) * splits + z) * 2;
            ml[0] = mrun[h];
            ml[1] = l_run[h];
        }
    }
}

// ---- tensor-core version for head_dim 64 and 128 -----------------------------------------
// The same block structure, but scores and the weighted sum are mma.sync m16n8k16 products:
// the (up to 8) query heads of the group are rows 0..7 of the 16-row A operand.  Each of the
// 4 warps owns 16 of a page's 64 keys and runs an online softmax of its own over them (no
// block-wide exchange per page); the four partial results are merged once at the end.
// K and V tiles are brought by TMA, one thread asking for a whole page, as halves of [64 tokens][64 dims] whose
// 16-byte chunks are swizzled by the row (128-byte swizzle), so ldmatrix reads them without bank conflicts; V is
// read with ldmatrix.trans.  (cp.async from all threads, 32 instructions per thread and page, kept an SM's two
// blocks busy for 0.7 us per page with issuing alone.)
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// c += a * b with rows 8..15 of a equal to zero (a1 = a3 = 0): only c[0], c[1] (rows 0..7) live on, the other two
// results are zero and are dropped
__device__ __forceinline__ void mma_rows8(float* c, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    [[maybe_unused]] float z2, z3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %10, %10};"
                 : "+f"(c[0]), "+f"(c[1]), "=f"(z2), "=f"(z3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
}

// Byte offset of element (row, col) in a tile of [64 rows][D] brought as D / 64 boxes with 128-byte swizzle: box
// col / 64, row of 128 bytes, its 16-byte chunk exchanged by the row's low three bits.
__device__ __forceinline__ uint32_t swz(int row, int col) {
    const int box = col >> 6, chunk = (col >> 3) & 7;
    return (uint32_t)(box * (PAGE * 128) + row * 128 + ((chunk ^ (row & 7)) << 4) + (col & 7) * 2);
}

// What the decode kernel starts from.  SRC_Q: q [T, H, D], rotated, and the cache already holds this step's
// keys and values.  SRC_QKV / SRC_PARTIALS: the output of the q/k/v product [T, (H + 2G) D], in bfloat16 or as
// the 32-bit partial sums [S][T][(H + 2G) D] of a product split over K (summed here in ascending s); the kernel
// then rotates q and k by the token's position itself (table of (cos, sin) as for `rope_append`), appends k and
// v to the cache and attends: one launch and no round trip of q through memory (model.py:197-211 in one kernel).
enum { SRC_Q = 0, SRC_QKV = 1, SRC_PARTIALS = 2 };

struct RopeSource {
    const void* src;          // qkv or its partial sums
    int S;                    // number of partial sums
    size_t slice;             // elements between partial sums
    const float* table;       // [table_len][D / 2][2]
    int table_len;
    int pairing;              // 0: pairs (2i, 2i+1); 1: pairs (i, i + D/2)
    int append;               // 0: the layer reads a cache another layer wrote
    const int* lengths_early; // optional: the lengths to request the first pages on before the preceding kernel has
                              // ended (null: the batch's own); they are checked against the batch's own afterwards
    int one_each;             // every sequence brings exactly one token: token t is sequence t (two loads fewer)
};

// x0[i], x1[i] = the elements e0[i], e1[i] of qkv for N pairs at once: from bfloat16, or as the sum of the S partial
// sums in ascending order.  The loads of eight partial sums (16 N values) are in flight together; a pair that is
// not wanted repeats a wanted one's addresses, so no branch sits between the loads.
template <int SRC, int N>
__device__ __forceinline__ void load_pairs(const RopeSource& r, const size_t* e0, const size_t* e1, float* x0, float* x1) {
    if (SRC == SRC_PARTIALS) {
        const float* p = (const float*)r.src;
#pragma unroll
        for (int i = 0; i < N; i++) { x0[i] = 0.f; x1[i] = 0.f; }
        constexpr int W = 8;                                  // partial sums in flight together
        for (int k = 0; k < r.S; k += W) {
            float a[W][N], c[W][N];
            if (r.pairing == 0) {                             // neighbours (e1 = e0 + 1, e0 even): one load of both
#pragma unroll
                for (int u = 0; u < W; u++) {
                    const float* pk = p + (size_t)min(k + u, r.S - 1) * r.slice;
#pragma unroll
                    for (int i = 0; i < N; i++) {
                        const float2 both = *reinterpret_cast<const float2*>(pk + e0[i]);
                        a[u][i] = both.x;
                        c[u][i] = both.y;
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < W; u++) {
                    const float* pk = p + (size_t)min(k + u, r.S - 1) * r.slice;
#pragma unroll
                    for (int i = 0; i < N; i++) { a[u][i] = pk[e0[i]]; c[u][i] = pk[e1[i]]; }
                }
            }
#pragma unroll
            for (int u = 0; u < W; u++)
                if (k + u < r.S) {
#pragma unroll
                    for (int i = 0; i < N; i++) { x0[i] += a[u][i]; x1[i] += c[u][i]; }
                }
        }
    } else {
        const __nv_bfloat16* p = (const __nv_bfloat16*)r.src;
        if (r.pairing == 0) {
#pragma unroll
            for (int i = 0; i < N; i++) {
                const float2 both = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + e0[i]));
                x0[i] = both.x;
                x1[i] = both.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < N; i++) { x0[i] = __bfloat162float(p[e0[i]]); x1[i] = __bfloat162float(p[e1[i]]); }
        }
    }
}

template <int D, int SRC, int DECODE_NBUF>
__global__ void __launch_bounds__(THREADS)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                       float* __restrict__ scratch_o, float* __restrict__ scratch_ml,
                       GfbPagedKV kv, GfbBatch b, int H, int G, float scale_log2e, int window, int splits, int* status,
                       RopeSource rs) {
    constexpr int PITCH = D + 8;                 // elements per row of q in shared memory
    constexpr int KSTEPS = D / 16, NT = D / 8;
    constexpr int HALF_BYTES = PAGE * 128;       // [64 tokens][64 dims]: one TMA box
    constexpr int TILE_BYTES = PAGE * D * 2;     // the keys (or values) of a page: D / 64 boxes
    constexpr int BOXES = 2 * D / 64;            // per page; each is asked for by another warp (at most THREADS / 32)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const uint32_t raw_u32 = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t tiles_u32 = (raw_u32 + 1023u) & ~1023u;     // swizzled boxes start on 1024-byte boundaries
    uint8_t* smem = smem_raw + (tiles_u32 - raw_u32);          // K0 V0 K1 V1 ... : DECODE_NBUF pairs
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem + 2 * DECODE_NBUF * TILE_BYTES);   // [8][PITCH]
    uint64_t* bars = reinterpret_cast<uint64_t*>(qs + 8 * PITCH);   // one barrier per tile pair: its page has arrived
    int* gave_up = reinterpret_cast<int*>(bars + DECODE_NBUF);      // a wait ran out: results are void, the status says so
    gfb_pdl_launch();
    const int rep = H / G;
    const int t = blockIdx.x, g = blockIdx.y, z = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, t4 = lane & 3;     // row (head) and column pair of the mma fragments
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
    if (tid == 0) {
        prefetch_map(&map_k);
        prefetch_map(&map_v);
#pragma unroll
        for (int i = 0; i < DECODE_NBUF; i++) mbar_init(bar0 + 8 * i, BOXES);
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Before the wait for the preceding kernel: what only depends on earlier steps.  The batch's bookkeeping and the
    // page table are written by the host before the step; the sequence's length is advanced by the last kernel of the
    // previous step, which has almost certainly ended, so the pages are requested on the length read now and the
    // length is read again behind the wait.
    const bool one_each = SRC != SRC_Q && rs.one_each != 0;
    const int s = one_each ? t : b.tok_seq[t];
    const int slot = b.slots[s];
    const int q_off = one_each ? 0 : t - b.cu_seqlens[s];
    const int* pt = kv.page_table + (size_t)slot * kv.max_pages;
    int pos, lo, first_page, last_page, per, p0, p1;
    auto plan = [&](int len) {
        pos = len + q_off;
        lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        first_page = lo / PAGE;
        last_page = pos / PAGE;
        const int n_pages = last_page - first_page + 1;
        per = (n_pages + splits - 1) / splits;
        p0 = first_page + z * per;
        p1 = min(last_page + 1, p0 + per);
    };
    bool bad_page = false;                       // uniform over the block
    int bad_index = 0;
    uint32_t parity_bits = 0, pending_bits = 0;  // per tile pair: the barrier phase to wait for; a page is on its way
    const uint64_t kv_policy = l2_evict_first_policy();
    // The page table's entries are read one request ahead of the copies that need them (an entry beyond the
    // sequence's pages is read but never used), so that no copy waits for a load of its address.
    auto entry = [&](int page_index) -> int {
        return (page_index >= 0 && page_index < kv.max_pages) ? __ldg(pt + page_index) : -1;
    };
    auto issue = [&](int page_index, int buf, int page) {
        if (page < 0 || page >= kv.n_pages) {
            bad_page = true;                     // reported once the length is certain
            bad_index = page_index;
            page = 0;
        }
        pending_bits |= 1u << buf;
        if (lane == 0 && warp < BOXES) {                     // one box per warp: its first lane announces and asks
            const uint32_t bar = bar0 + 8 * buf;
            const int y = (page * G + g) * PAGE;             // the page's first row in the pool seen as [rows][D]
            mbar_expect_tx(bar, HALF_BYTES);
            // boxes in the order they lie in shared memory: the key tile's halves, then the value tile's
            tma_load_2d_hint(tiles_u32 + 2 * buf * TILE_BYTES + warp * HALF_BYTES, warp < D / 64 ? &map_k : &map_v,
                             (warp % (D / 64)) * 64, y, bar, kv_policy);
        }
    };
    // Waits for the page of a tile pair, a second at most (then the status tells, and the block goes on without waiting
    // any longer).  All threads wait: each must see the copy's bytes itself.
    auto wait_page = [&](int buf) {
        const uint32_t bar = bar0 + 8 * buf, parity = (parity_bits >> buf) & 1u;
        bool there = mbar_try_wait(bar, parity) != 0;
        if (!there) {
            const unsigned long long t0 = global_ns();
            while (!there) {
#pragma unroll 1
                for (int i = 0; i < 64 && !there; i++) there = mbar_try_wait(bar, parity) != 0;
                if (there) break;
                if (*reinterpret_cast<volatile int*>(gave_up)) break;
                if (global_ns() - t0 > PAGE_WAIT_LIMIT_NS) {
                    if (atomicExch(gave_up, 1) == 0) gfb_report(status, GFB_ERR_WAIT_TIMEOUT, 300 + buf, (int)(blockIdx.x + gridDim.x * blockIdx.y));
                    break;
                }
            }
        }
        if (there) {
            parity_bits ^= 1u << buf;
            pending_bits &= ~(1u << buf);
        }
    };
    // A block that is its sequence's only slice and has no window starts at the table's first entry whatever the
    // length is: its entries are then asked for together with the length, not behind it.
    const bool from_zero = splits == 1 && window <= 0;
    int ahead[DECODE_NBUF];                      // entries ahead_first .. ahead_first + DECODE_NBUF - 1
    int ahead_first = -1;
    auto entries_ahead = [&](int first) {
        ahead_first = first;
#pragma unroll
        for (int a = 0; a < DECODE_NBUF; a++) ahead[a] = entry(first + a);
    };
    int next_entry = -1;                         // of page p + DECODE_NBUF - 1 while page p is worked on
    // DECODE_NBUF - 1 pages in flight while q is prepared and, later, while a page is worked on
    auto first_pages = [&]() {
        if (ahead_first != p0) entries_ahead(p0);
#pragma unroll
        for (int a = 0; a < DECODE_NBUF - 1; a++)
            if (p0 + a < p1) issue(p0 + a, a, ahead[a]);
        next_entry = ahead[DECODE_NBUF - 1];
    };
    // Only a kernel that appends may ask for pages this early: it patches its own token's row into the copy of the
    // last page, and all other rows were written in earlier steps.  A kernel that reads what ANOTHER kernel of this
    // step stores (SRC_Q behind the rotary/append kernel; append == 0 behind the cache entry's owner) must not copy
    // a page before that store has landed, so it asks behind the wait.
    const bool early = SRC != SRC_Q && rs.append != 0;        // uniform over the grid
    constexpr int half = D / 2;
    constexpr int IT = 8 * half / THREADS;                    // q pairs per thread; one more pair for k or v
    // (cos, sin) of the token's position for this thread's pairs of q and of k, and the table entry of the page that
    // takes the new key and value: asked for as soon as a position is known, and again if it was another one
    float2 csq[IT], csk;
    int cs_pos = -2, last_entry = -1;
    auto position_loads = [&]() {
        cs_pos = pos;
        const bool in_table = pos >= 0 && pos < rs.table_len;
        const float* row = rs.table + (size_t)(in_table ? pos : 0) * half * 2;
#pragma unroll
        for (int it = 0; it < IT; it++) csq[it] = __ldg(reinterpret_cast<const float2*>(row + 2 * ((tid + it * THREADS) % half)));
        csk = __ldg(reinterpret_cast<const float2*>(row + 2 * (tid % half)));
        last_entry = entry(last_page);
    };
    int len_early = 0;
    if (early) {
        if (from_zero) entries_ahead(0);
        len_early = __ldcg((rs.lengths_early ? rs.lengths_early : b.lengths) + slot);
        plan(len_early);
        first_pages();
        position_loads();
    }
    gfb_pdl_wait();
    const int len_now = __ldcg(b.lengths + slot);
    if (!early) {
        len_early = len_now;
        plan(len_now);
        first_pages();
        if (SRC != SRC_Q) position_loads();
    }
    // SRC != SRC_Q: the new key and value of this token, kept in registers by the threads that made them.  The
    // slice that owns the last page patches them into its shared-memory copy of that page: the page may have
    // been read before the store to the cache landed.
    bool patch = false;
    int off = 0, new_i0 = 0, new_i1 = 1;
    __nv_bfloat16 new0 = __float2bfloat16_rn(0.f), new1 = new0;
    // the length was another one after all: drop what was requested and start again (uniform over the block)
    auto settle_length = [&]() {
        if (len_now != len_early) {
#pragma unroll
            for (int a = 0; a < DECODE_NBUF - 1; a++)
                if (pending_bits >> a & 1u) wait_page(a);
            __syncthreads();
            bad_page = false;
            plan(len_now);
            first_pages();
        }
    };
    if (SRC == SRC_Q) {
        for (int i = tid; i < 8 * D; i += THREADS) {
            int row = i / D, col = i - row * D;
            qs[row * PITCH + col] = row < rep ? q[((size_t)t * H + g * rep + row) * D + col] : __float2bfloat16_rn(0.f);
        }
        settle_length();
    } else {
        const size_t W = (size_t)(H + 2 * G) * D;
        size_t e0[IT + 1], e1[IT + 1];
        int qi0[IT], qi1[IT], qrow[IT], qi[IT];
#pragma unroll
        for (int it = 0; it < IT; it++) {
            const int idx = tid + it * THREADS;
            qrow[it] = idx / half;
            qi[it] = idx - qrow[it] * half;
            qi0[it] = rs.pairing == 1 ? qi[it] : 2 * qi[it];
            qi1[it] = rs.pairing == 1 ? qi[it] + half : 2 * qi[it] + 1;
            const size_t e = (size_t)t * W + (size_t)(g * rep + (qrow[it] < rep ? qrow[it] : 0)) * D;
            e0[it] = e + qi0[it];
            e1[it] = e + qi1[it];
        }
        const bool is_key = tid < half;
        const int ki = is_key ? tid : tid - half;
        if (tid < 2 * half) {                                     // the threads that hold a pair of the new key or value
            new_i0 = (is_key && rs.pairing == 1) ? ki : 2 * ki;
            new_i1 = (is_key && rs.pairing == 1) ? ki + half : 2 * ki + 1;
            const size_t e = (size_t)t * W + (size_t)(is_key ? H + g : H + G + g) * D;
            e0[IT] = e + new_i0;
            e1[IT] = e + new_i1;
        } else {
            e0[IT] = e0[0];
            e1[IT] = e1[0];
        }
        float x0[IT + 1], x1[IT + 1];
        load_pairs<SRC, IT + 1>(rs, e0, e1, x0, x1);
        settle_length();                                           // from here on the position is certain
        if (cs_pos != pos) position_loads();
        const bool ok = pos >= 0 && pos < rs.table_len;
        if (!ok && tid == 0 && g == 0 && z == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
        const int n_all = last_page - first_page + 1;
        const int z_last = (n_all - 1) / per;
        int page = -1;
        if (rs.append && ok && z == z_last) {
            off = pos - last_page * PAGE;
            page = last_entry;
            if (page < 0 || page >= kv.n_pages) {
                if (tid == 0) gfb_report(status, GFB_ERR_CACHE_RANGE, t, pos);
                page = -1;
            }
        }
        patch = page >= 0 && tid < 2 * half;
#pragma unroll
        for (int it = 0; it < IT; it++) {
            const float2 cs = csq[it];
            const bool live = ok && qrow[it] < rep;
            qs[qrow[it] * PITCH + qi0[it]] = __float2bfloat16_rn(live ? x0[it] * cs.x - x1[it] * cs.y : 0.f);
            qs[qrow[it] * PITCH + qi1[it]] = __float2bfloat16_rn(live ? x1[it] * cs.x + x0[it] * cs.y : 0.f);
        }
        if (patch) {
            const size_t dst = (((size_t)page * G + g) * PAGE + off) * D;
            if (is_key) {                                     // the key: rotated
                const float2 cs = csk;
                new0 = __float2bfloat16_rn(x0[IT] * cs.x - x1[IT] * cs.y);
                new1 = __float2bfloat16_rn(x1[IT] * cs.x + x0[IT] * cs.y);
            } else {                                          // the value: copied
                new0 = __float2bfloat16_rn(x0[IT]);
                new1 = __float2bfloat16_rn(x1[IT]);
            }
            __nv_bfloat16* dp = (__nv_bfloat16*)(is_key ? kv.k_pool : kv.v_pool) + dst;
            dp[new_i0] = new0;
            dp[new_i1] = new1;
        }
    }
    __syncthreads();                                           // qs complete

    uint32_t qa[KSTEPS][2];
#pragma unroll
    for (int k = 0; k < KSTEPS; k++) {
        qa[k][0] = *reinterpret_cast<const uint32_t*>(qs + gq * PITCH + k * 16 + 2 * t4);
        qa[k][1] = *reinterpret_cast<const uint32_t*>(qs + gq * PITCH + k * 16 + 8 + 2 * t4);
    }
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;
    const int mid = lane >> 3, mr = lane & 7;                  // ldmatrix: this lane addresses row mr of matrix mid

    for (int p = p0; p < p1; p++) {
        const int buf = (p - p0) % DECODE_NBUF;
        if (p + DECODE_NBUF - 1 < p1) issue(p + DECODE_NBUF - 1, (p - p0 + DECODE_NBUF - 1) % DECODE_NBUF, next_entry);
        next_entry = entry(p + DECODE_NBUF);                   // in flight while this page is worked on
        wait_page(buf);
        if (SRC != SRC_Q && p == last_page) {                  // uniform: the block's last page holds the new token
            if (patch) {
                uint8_t* tile = smem + (2 * buf + (tid < half ? 0 : 1)) * TILE_BYTES;
                *reinterpret_cast<__nv_bfloat16*>(tile + swz(off, new_i0)) = new0;
                *reinterpret_cast<__nv_bfloat16*>(tile + swz(off, new_i1)) = new1;
            }
            __syncthreads();
        }
        const uint32_t kbase = tiles_u32 + 2 * buf * TILE_BYTES;
        const uint32_t vbase = kbase + TILE_BYTES;

        // scores of this warp's 16 keys (two n-tiles of 8) for rows = heads
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; n++) { sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f; }
#pragma unroll
        for (int k = 0; k < KSTEPS; k++) {
            // matrices: (keys 0-7, dims lo), (keys 0-7, dims hi), (keys 8-15, dims lo), (keys 8-15, dims hi)
            uint32_t addr = kbase + swz(warp * 16 + (mid >> 1) * 8 + mr, k * 16 + (mid & 1) * 8);
            uint32_t b0, b1, b2, b3;
            ldsm_x4(addr, b0, b1, b2, b3);
            mma_rows8(sc[0], qa[k][0], qa[k][1], b0, b1);
            mma_rows8(sc[1], qa[k][0], qa[k][1], b2, b3);
        }
        // mask, online softmax over this warp's keys (row = head gq, columns 2*t4, 2*t4+1 of each n-tile)
        float v[4];
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                int j = p * PAGE + warp * 16 + n * 8 + 2 * t4 + e;
                float x = (j >= lo && j <= pos) ? sc[n][e] * scale_log2e : -INFINITY;
                v[n * 2 + e] = x;
                mx = fmaxf(mx, x);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        float corr = 1.f, pr[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
#pragma unroll
            for (int e = 0; e < 4; e++) pr[e] = (v[e] == -INFINITY) ? 0.f : exp2f(v[e] - m_new);
        }
        float rs = pr[0] + pr[1] + pr[2] + pr[3];
        rs += __shfl_xor_sync(0xffffffffu, rs, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        l_run = l_run * corr + rs;
        m_run = m_new;
        const uint32_t pa0 = pack2(pr[0], pr[1]), pa2 = pack2(pr[2], pr[3]);
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
            o[j][0] *= corr; o[j][1] *= corr; o[j + 1][0] *= corr; o[j + 1][1] *= corr;
            // matrices: (keys 0-7, dims j), (keys 8-15, dims j), (keys 0-7, dims j+1), (keys 8-15, dims j+1)
            uint32_t addr = vbase + swz(warp * 16 + (mid & 1) * 8 + mr, (j + (mid >> 1)) * 8);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(addr, b0, b1, b2, b3);
            mma_rows8(o[j], pa0, pa2, b0, b1);
            mma_rows8(o[j + 1], pa0, pa2, b2, b3);
        }
        __syncthreads();                                       // this buffer is refilled next round
    }
    if (pending_bits) {                                        // only after a wait that ran out: once more, then leave
#pragma unroll
        for (int a = 0; a < DECODE_NBUF; a++)
            if (pending_bits >> a & 1u) wait_page(a);
    }
    if (bad_page && tid == 0) gfb_report(status, GFB_ERR_PAGE_TABLE, slot, bad_index);

    // Merge of the four warps' partial softmaxes; the tile area is free now.  The warps exchange (max, sum) first, each
    // scales its own sums in registers to the common maximum (and, with one slice, by 1 / the whole sum), and the block
    // adds the four scaled copies.
    constexpr int OP = D + 8;                                  // floats per row: the rows of a store fall on different banks
    float* Ow = (float*)smem;                                  // [4][8][OP]
    float* mw = Ow + 4 * 8 * OP;                               // [4][8]
    float* lw = mw + 32;                                       // [4][8]
    if (t4 == 0) { mw[warp * 8 + gq] = m_run; lw[warp * 8 + gq] = l_run; }
    __syncthreads();
    const float m_all = fmaxf(fmaxf(mw[gq], mw[8 + gq]), fmaxf(mw[16 + gq], mw[24 + gq]));
    float l_all = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const float mm = mw[w * 8 + gq];
        if (mm != -INFINITY) l_all += lw[w * 8 + gq] * exp2f(mm - m_all);
    }
    float f = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_all);
    if (splits == 1) f = l_all > 0.f ? f / l_all : 0.f;
#pragma unroll
    for (int j = 0; j < NT; j++)
        *reinterpret_cast<float2*>(Ow + (warp * 8 + gq) * OP + j * 8 + 2 * t4) = make_float2(o[j][0] * f, o[j][1] * f);
    if (splits > 1 && warp == 0 && t4 == 0 && gq < rep) {
        float* ml = scratch_ml + (((size_t)t * H + g * rep + gq) * splits + z) * 2;
        ml[0] = m_all;
        ml[1] = l_all;
    }
    __syncthreads();
    for (int idx = tid; idx < rep * (D / 2); idx += THREADS) {
        const int h = idx / (D / 2), dim = 2 * (idx - h * (D / 2));
        float2 acc = *reinterpret_cast<const float2*>(Ow + h * OP + dim);
#pragma unroll
        for (int w = 1; w < 4; w++) {
            const float2 a = *reinterpret_cast<const float2*>(Ow + (w * 8 + h) * OP + dim);
            acc.x += a.x;
            acc.y += a.y;
        }
        const int head = g * rep + h;
        if (splits == 1)
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * H + head) * D + dim) = __floats2bfloat162_rn(acc.x, acc.y);
        else
            *reinterpret_cast<float2*>(scratch_o + (((size_t)t * H + head) * splits + z) * D + dim) = acc;
    }
}

__global__ void attn_combine_kernel(const float* __restrict__ scratch_o, const float* __restrict__ scratch_ml,
                                    __nv_bfloat16* __restrict__ out, int H, int d, int splits) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int t = blockIdx.x, head = blockIdx.y;
    const float* ml = scratch_ml + ((size_t)t * H + head) * splits * 2;
    float m = -INFINITY;
    for (int z = 0; z < splits; z++) m = fmaxf(m, ml[2 * z]);
    float l = 0.f;
    for (int z = 0; z < splits; z++) l += (ml[2 * z] == -INFINITY) ? 0.f : ml[2 * z + 1] * exp2f(ml[2 * z] - m);
    float inv = l > 0.f ? 1.f / l : 0.f;
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < splits; z++) {
            if (ml[2 * z] == -INFINITY) continue;
            o += scratch_o[(((size_t)t * H + head) * splits + z) * d + dim] * exp2f(ml[2 * z] - m);
        }
        out[((size_t)t * H + head) * d + dim] = __float2bfloat16_rn(o * inv);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Launch of the tensor-core decode kernel for head_dim 64 or 128 and one of the three sources: the tile pairs, the
// query rows and the barriers of shared memory; the merge area reuses the tiles.
cudaError_t launch_decode_mma(int d, int src, dim3 grid, cudaStream_t stream, const void* q, void* out, float* so, float* sml,
                              GfbPagedKV kv, GfbBatch b, int H, int G, float scale, int window, int splits, int* status,
                              RopeSource rs, int pages_per_slice) {
    typedef void (*Kern)(const CUtensorMap, const CUtensorMap, const __nv_bfloat16*, __nv_bfloat16*, float*, float*, GfbPagedKV,
                         GfbBatch, int, int, float, int, int, int*, RopeSource);
    // Tile pairs per block: five where the grid covers at most a quarter of the SMs (a short context is then requested
    // all at once; with more blocks than that, one block of five pairs per SM leaves no room for the blocks of the
    // product behind it, which want to fetch their weights meanwhile: 8 sequences x 8 heads, 2.99 -> 2.92 ms per step);
    // two where more than two blocks per SM wait with a few pages each (three blocks then fit an SM, which saves a
    // round of blocks between two and three per SM: 48 sequences x 8 heads of 200 tokens, 12.0 -> 8.1 us; and their
    // set-ups and merges overlap: 40 heads of their own keys at batch 32, 42 -> 38 us; 8 groups at batch 64 and 150
    // tokens, 14.5 -> 12.6 us); three otherwise (long slices want two pages in flight behind the one being worked on).
    static const Kern kerns[3][2][3] = {
        {{attn_decode_mma_kernel<64, SRC_Q, DECODE_NBUF_MANY>, attn_decode_mma_kernel<64, SRC_QKV, DECODE_NBUF_MANY>,
          attn_decode_mma_kernel<64, SRC_PARTIALS, DECODE_NBUF_MANY>},
         {attn_decode_mma_kernel<128, SRC_Q, DECODE_NBUF_MANY>, attn_decode_mma_kernel<128, SRC_QKV, DECODE_NBUF_MANY>,
          attn_decode_mma_kernel<128, SRC_PARTIALS, DECODE_NBUF_MANY>}},
        {{attn_decode_mma_kernel<64, SRC_Q, DECODE_NBUF_FEW>, attn_decode_mma_kernel<64, SRC_QKV, DECODE_NBUF_FEW>,
          attn_decode_mma_kernel<64, SRC_PARTIALS, DECODE_NBUF_FEW>},
         {attn_decode_mma_kernel<128, SRC_Q, DECODE_NBUF_FEW>, attn_decode_mma_kernel<128, SRC_QKV, DECODE_NBUF_FEW>,
          attn_decode_mma_kernel<128, SRC_PARTIALS, DECODE_NBUF_FEW>}},
        {{attn_decode_mma_kernel<64, SRC_Q, DECODE_NBUF_SHORT>, attn_decode_mma_kernel<64, SRC_QKV, DECODE_NBUF_SHORT>,
          attn_decode_mma_kernel<64, SRC_PARTIALS, DECODE_NBUF_SHORT>},
         {attn_decode_mma_kernel<128, SRC_Q, DECODE_NBUF_SHORT>, attn_decode_mma_kernel<128, SRC_QKV, DECODE_NBUF_SHORT>,
          attn_decode_mma_kernel<128, SRC_PARTIALS, DECODE_NBUF_SHORT>}}};
    static bool configured[3][2][3] = {};
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    }
    const int di = d == 128 ? 1 : 0;
    const long blocks = (long)grid.x * grid.y * grid.z;
    const int few = blocks <= sms / 4 ? 1 : (blocks > 2L * sms && pages_per_slice > 0 && pages_per_slice <= 6) ? 2 : 0;
    const int nbuf = few == 1 ? DECODE_NBUF_FEW : few == 2 ? DECODE_NBUF_SHORT : DECODE_NBUF_MANY;
    // alignment slack, tiles, q rows, barriers and a flag
    const size_t msmem = 1024 + (size_t)2 * nbuf * PAGE * d * 2 + (size_t)8 * (d + 8) * 2 + 8 * nbuf + 16;
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        gfb_fail("decode attention: the driver does not export cuTensorMapEncodeTiled");
        return cudaErrorInvalidValue;
    }
    if ((long long)kv.n_pages * G * PAGE > 2147483647LL) {       // TMA coordinates are 32-bit
        gfb_fail("decode attention: %d pages x %d heads x %d tokens do not fit the 32-bit row coordinate of a tensor map",
                 kv.n_pages, G, PAGE);
        return cudaErrorInvalidValue;
    }
    CUtensorMap mk, mv;
    for (int i = 0; i < 2; i++) {                            // a pool seen as [pages x heads x 64 rows][d]
        cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)kv.n_pages * G * PAGE};
        cuuint64_t strides[1] = {(cuuint64_t)d * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)PAGE};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(i ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(i ? kv.v_pool : kv.k_pool), dims,
                         strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            gfb_fail("decode attention: tensor map of the cache refused (%d): %d pages, %d heads, head_dim %d, pool at %p",
                     (int)r, kv.n_pages, G, d, i ? kv.v_pool : kv.k_pool);
            return cudaErrorInvalidValue;
        }
    }
    Kern kern = kerns[few][di][src];
    if (msmem > 48 * 1024 && !configured[few][di][src]) {
        cudaError_t a = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)msmem);
        if (a != cudaSuccess) {
            gfb_fail("decode attention: %zu bytes of shared memory refused: %s", msmem, cudaGetErrorString(a));
            return cudaErrorInvalidValue;
        }
        configured[few][di][src] = true;
    }
    gfb_error_text[0] = 0;
    return gfb_launch(kern, grid, dim3(THREADS), msmem, stream, mk, mv, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, so, sml, kv, b,
                      H, G, scale * 1.4426950408889634f, window, splits, status, rs);
}

}  // namespace

// Bytes of scratch the decode kernel needs for `splits` > 1: [T, H, splits, d + 2] floats.
GFB_API long gfb_attn_decode_scratch_bytes(int T, int H, int d, int splits) {
    return splits > 1 ? (long)T * H * splits * (d + 2) * 4 : 0;
}

GFB_API int gfb_attn_decode(const void* q, void* out, void* k_pool, void* v_pool, const int* page_table, int max_pages,
                            int page_size, int n_pages, const int* cu_seqlens, const int* tok_seq, const int* slots,
                            const int* lengths, int n_seqs, int n_tokens, int H, int G, int d, float scale, int window,
                            int splits, float* scratch, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (page_size != PAGE) return gfb_fail("gfb_attn_decode: pages of %d tokens (the kernel is built for %d)", page_size, PAGE);
    if (d % 8 || d > THREADS * MAX_DPT) return gfb_fail("gfb_attn_decode: head_dim %d must be a multiple of 8, at most %d", d, THREADS * MAX_DPT);
    if (G <= 0 || H % G || H / G > MAX_REP) return gfb_fail("gfb_attn_decode: %d heads over %d groups (at most %d per group)", H, G, MAX_REP);
    if (splits < 1 || G > 65535 || splits > 65535) return gfb_fail("gfb_attn_decode: bad split count %d", splits);
    if (splits > 1 && scratch == nullptr) return gfb_fail("gfb_attn_decode: %d slices need scratch memory", splits);
    const int rep = H / G;
    size_t smem = (size_t)4 * PAGE * d * 2 + (size_t)rep * d * 4 + (size_t)rep * PAGE * 4;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("gfb_attn_decode: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    float* so = scratch;
    float* sml = scratch ? scratch + (size_t)n_tokens * H * splits * d : nullptr;
    dim3 grid(n_tokens, G, splits);
    cudaError_t e;
    if (d == 128 || d == 64) {
        e = launch_decode_mma(d, SRC_Q, grid, stream, q, out, so, sml, kv, b, H, G, scale, window, splits, status, RopeSource{}, 0);
        if (e == cudaErrorInvalidValue && gfb_error_text[0]) return 1;
    } else {
        e = gfb_launch(attn_decode_kernel, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q,
                       (__nv_bfloat16*)out, so, sml, kv, b, H, G, d, scale * 1.4426950408889634f, window, splits, status);
    }
    if (gfb_check(e, "gfb_attn_decode")) return 1;
    if (splits > 1) {
        dim3 cgrid(n_tokens, H);
        e = gfb_launch(attn_combine_kernel, cgrid, dim3(128), 0, stream, (const float*)so, (const float*)sml,
                       (__nv_bfloat16*)out, H, d, splits);
        return gfb_check(e, "gfb_attn_decode (combine)");
    }
    return 0;
}

// Rotary encoding, cache append and decode attention in one launch (head_dim 64 or 128, bfloat16): `src` is the
// q/k/v product [T, (H + 2G) d] in bfloat16 (n_part = 0) or its n_part 32-bit partial sums [n_part][T][(H + 2G) d].
// With append = 0 only q is taken from it (the layer reads a cache that another layer wrote).
// The kernel asks for its first pages before the preceding kernel has ended, on the lengths as they are then, and
// reads the lengths again afterwards; lengths_early (optional, per slot like lengths) stands in for the first read,
// which lets a test make the two differ.  Every sequence brings at most one token (a second one would attend to a key
// that this launch has not stored yet).  max_kv_len (0: unknown): the longest sequence of the batch after this step,
// as the host knows it; it only chooses how many pages a block keeps in flight.
GFB_API int gfb_attn_decode_rope(const void* src, int n_part, void* out, void* k_pool, void* v_pool, const int* page_table,
                                 int max_pages, int page_size, int n_pages, const int* cu_seqlens, const int* tok_seq,
                                 const int* slots, const int* lengths, int n_seqs, int n_tokens, const float* table,
                                 int table_len, int H, int G, int d, int pairing, int append, float scale, int window,
                                 int splits, float* scratch, int* status, const int* lengths_early, int max_kv_len,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (page_size != PAGE) return gfb_fail("gfb_attn_decode_rope: pages of %d tokens (the kernel is built for %d)", page_size, PAGE);
    if (d != 64 && d != 128) return gfb_fail("gfb_attn_decode_rope: head_dim %d (64 or 128)", d);
    if (G <= 0 || H % G || H / G > MAX_REP) return gfb_fail("gfb_attn_decode_rope: %d heads over %d groups (at most %d per group)", H, G, MAX_REP);
    if (splits < 1 || G > 65535 || splits > 65535) return gfb_fail("gfb_attn_decode_rope: bad split count %d", splits);
    if (splits > 1 && scratch == nullptr) return gfb_fail("gfb_attn_decode_rope: %d slices need scratch memory", splits);
    if (pairing != 0 && pairing != 1) return gfb_fail("gfb_attn_decode_rope: unknown pairing %d", pairing);
    if ((uintptr_t)src % 8) return gfb_fail("gfb_attn_decode_rope: the q/k/v product must start on an 8-byte boundary");
    GfbPagedKV kv{k_pool, v_pool, page_table, max_pages, page_size, n_pages};
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    float* so = scratch;
    float* sml = scratch ? scratch + (size_t)n_tokens * H * splits * d : nullptr;
    RopeSource rs{src, n_part, (size_t)n_tokens * (H + 2 * G) * d, table, table_len, pairing, append, lengths_early,
                  n_tokens == n_seqs ? 1 : 0};
    const int pages = max_kv_len > 0 ? (max_kv_len + PAGE - 1) / PAGE : 0;
    cudaError_t e = launch_decode_mma(d, n_part > 0 ? SRC_PARTIALS : SRC_QKV, dim3(n_tokens, G, splits), stream, nullptr, out, so, sml,
                                      kv, b, H, G, scale, window, splits, status, rs, (pages + splits - 1) / splits);
    if (e == cudaErrorInvalidValue && gfb_error_text[0]) return 1;
    if (gfb_check(e, "gfb_attn_decode_rope")) return 1;
    if (splits > 1) {
        e = gfb_launch(attn_combine_kernel, dim3(n_tokens, H), dim3(128), 0, stream, (const float*)so, (const float*)sml,
                       (__nv_bfloat16*)out, H, d, splits);
        return gfb_check(e, "gfb_attn_decode_rope (combine)");
    }
    return 0;
}

// ---- the entry point that allocates nothing (see attn_decode_noalloc.h) -----------------
#include "attn_decode_noalloc.h"

// Scratch of the split-KV partials for callers that cannot allocate.  In host code this name is
// only a handle for the runtime, not a device address: its address is looked up once per device.
static __device__ __align__(256) float gfb_noalloc_scratch[GFB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* noalloc_scratch_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}

GFB_API int gfb_attn_decode_noalloc(const void* q, void* out, void* k_pool, void* v_pool, const int* page_table,
                                    int max_pages, int page_size, int n_pages, const int* cu_seqlens, const int* tok_seq,
                                    const int* slots, const int* lengths, int n_seqs, int n_tokens, int H, int G, int d,
                                    float scale, int window, int splits, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (splits < 1 || H <= 0 || d <= 0) return gfb_fail("gfb_attn_decode_noalloc: bad sizes (H %d, d %d, splits %d)", H, d, splits);
    float* scratch = nullptr;
    if (splits > 1) {
        long long need = (long long)n_tokens * H * splits * (d + 2);
        if (need > (long long)GFB_NOALLOC_SCRATCH_FLOATS)
            return gfb_fail("gfb_attn_decode_noalloc: %d tokens x %d heads x %d slices x (%d + 2) = %lld floats of scratch "
                            "exceed the built-in %d; use fewer slices or gfb_attn_decode with your own scratch",
                            n_tokens, H, splits, d, need, GFB_NOALLOC_SCRATCH_FLOATS);
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return gfb_fail("gfb_attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
        if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return gfb_fail("gfb_attn_decode_noalloc: device %d out of range", dev);
        if (noalloc_scratch_ptr[dev] == nullptr) {          // set-up, once per device, with that device current
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, gfb_noalloc_scratch);
            if (e != cudaSuccess || p == nullptr)
                return gfb_fail("gfb_attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            noalloc_scratch_ptr[dev] = p;
        }
        scratch = noalloc_scratch_ptr[dev];
    }
    return gfb_attn_decode(q, out, k_pool, v_pool, page_table, max_pages, page_size, n_pages, cu_seqlens, tok_seq, slots,
                           lengths, n_seqs, n_tokens, H, G, d, scale, window, splits, scratch, status, stream);
}

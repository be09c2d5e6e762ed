// Prefill attention on the 5th-generation tensor cores (tcgen05), head_dim 128 or 64, bfloat16.
//
// Causal attention of a run of new tokens over the paged cache (gpt-fast: the
// SDPA call of model.py:209-211).  A block owns one key/value head and a tile of
// TQ = 128 / (heads per group) consecutive query tokens of one sequence (rounded down: 42 tokens
// and 126 rows for 3 heads per group); its rows are the (token, head of the group) pairs, one per
// tensor-memory lane.
// Keys and values are visited 128 at a time (two pages of 64):
//
//   S = Q K^T        tcgen05.mma, A = Q and B = K from shared memory (TMA, 128B swizzle),
//                    S (32-bit) in tensor memory, two buffers
//   softmax          4 warps, one row per thread: tcgen05.ld of S, running maximum and sum
//                    in 32-bit registers, P rounded to bfloat16 and stored back into
//                    tensor memory (tcgen05.st); the reference maximum follows the true one
//                    lazily (steps of 2^8), and only then O is rescaled in tensor memory
//   O += P V         tcgen05.mma with A = P from tensor memory and B = V from shared
//                    memory as an MN-major operand (V lies [key][dim] in the cache)
//
// The MMA warp issues S of the next 128 keys before it waits for P of the current
// ones, so the tensor cores work while the softmax warps do.  Warp 0 is the TMA
// producer (Q once through a 3-D map over [token, head, dim] that lays the rows out
// as (token, head of group); K and V pages through 2-D maps over the pools), warp 1
// allocates tensor memory and issues the MMAs, warps 2..5 are the softmax and
// epilogue warps.  Every wait is bounded by wall-clock time (see gemm_tc.cu).
#include "common.cuh"

#include <cuda.h>

GFB_DEFINE_LAST_ERROR()

namespace {

constexpr int D = 128;                    // head_dim
constexpr int PAGE = 64;
constexpr int ROWS = 128;                 // query rows per block
constexpr int KEYS = 128;                 // keys per iteration (two pages)
constexpr int HALF_BYTES = 128 * 128;     // 128 rows x 64 elements x 2 bytes: one swizzled half tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;
constexpr int KV_STAGES = 2;
static_assert(KV_STAGES == 2, "the one-tile kernel frees K/V stage s by the barriers of score buffer s");
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// tensor-memory columns
constexpr uint32_t COL_S = 0;             // two score buffers of 128 columns
constexpr uint32_t COL_O = 256;           // output accumulator, 128 columns
constexpr uint32_t COL_P = 384;           // two probability buffers of 64 columns (bfloat16 pairs)

struct Bars {
    unsigned long long q_full, q_empty, o_free;
    unsigned long long k_full[KV_STAGES];     // (a K stage is free again when the scores of its block are done: s_full,
    unsigned long long v_full[KV_STAGES];     //  a V stage when its P V is: pv_done; a commit per barrier costs MMA issue time)
    unsigned long long s_full[2], s_empty[2];
    unsigned long long p_ready;
    unsigned long long pv_done[2];            // P V of the even / odd key blocks has landed
    unsigned long long o_full;                // the item's last P V has landed (one phase per item)
    unsigned long long xch[4];                // per quarter of the rows: both warps of a row have written their half's maximum
    unsigned long long fin[4];                // the same for their sums at the end of an item
    uint32_t tmem_base;
    int abort_flag;
    float mx_half[2][2][ROWS];                // [key block parity][half][row]
    float l_half[2][2][ROWS];                 // [item parity][half][row]
};

// The first TMA copy through a tensor map fetches the 128-byte map; asking for it at once hides that behind the
// block's set-up.
__device__ __forceinline__ void prefetch_map(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int which) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 128; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            gfb_report(status, GFB_ERR_WAIT_TIMEOUT, 100 + which, (int)(blockIdx.x + gridDim.x * blockIdx.y));
            return false;
        }
        __nanosleep(64);
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// K-major operand tile with 128-byte swizzle (rows of 128 bytes, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand tile with 128-byte swizzle: rows are K (keys), 64 MN elements (dims) per 128-byte
// row; 8-row groups 1024 bytes apart (stride offset), the next 64 dims one half tile further (leading offset)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(HALF_BYTES >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
// The same load without the wait, and the wait as a separate step that names the registers, so that the compiler
// keeps every use of them behind it: several loads can then be in flight before one wait.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait32(uint32_t* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :: "memory");
}
// a whole row of 128 scores: four loads in flight, then the wait
__device__ __forceinline__ void tmem_ld_row128(uint32_t taddr, float (*v)[32]) {
    uint32_t r[4][32];
#pragma unroll
    for (int c = 0; c < 4; c++) tmem_ld32_issue(taddr + c * 32, r[c]);
#pragma unroll
    for (int c = 0; c < 4; c++) tmem_ld_wait32(r[c]);
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
        for (int i = 0; i < 32; i++) v[c][i] = __uint_as_float(r[c][i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// two 32-bit lanes per instruction (sm_100): r = a * b + c and r = a + b on pairs; the maximum of three
__device__ __forceinline__ void fma2(float a0, float a1, float b, float c, float& r0, float& r1) {
    unsigned long long pa, pb, pc, pr;
    asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(pb) : "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(pc) : "f"(c));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pr) : "l"(pa), "l"(pb), "l"(pc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r0), "=f"(r1) : "l"(pr));
}
__device__ __forceinline__ void add2(float& a0, float& a1, float b0, float b1) {
    unsigned long long pa, pb;
    asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(pb) : "f"(b0), "f"(b1));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(pa) : "l"(pa), "l"(pb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(pa));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// One (sequence, tile of TQ query tokens, key/value head) unit of work.
struct TileWork {
    int seq, tq0, g;
    int t_first, nq, slot, pos0, last_pos, first_lo, blk0, n_iter, last_page;
};
// Work item w of the grid's list (long tiles first: the tile index runs backwards); false: an empty item.
__device__ __forceinline__ bool tile_work(const GfbBatch& b, int w, int n_x, int G, int TQ, int window, TileWork& t) {
    const int xi = w / G;
    t.g = w - xi * G;
    t.seq = -1;
    int left = n_x - 1 - xi;
    for (int i = 0; i < b.n_seqs; i++) {
        const int qlen = b.cu_seqlens[i + 1] - b.cu_seqlens[i];
        const int nt = (qlen + TQ - 1) / TQ;
        if (left < nt) { t.seq = i; t.tq0 = left * TQ; break; }
        left -= nt;
    }
    if (t.seq < 0) return false;
    t.t_first = b.cu_seqlens[t.seq];
    const int qlen = b.cu_seqlens[t.seq + 1] - t.t_first;
    t.nq = min(TQ, qlen - t.tq0);
    t.slot = b.slots[t.seq];
    t.pos0 = b.lengths[t.slot] + t.tq0;
    t.last_pos = t.pos0 + t.nq - 1;
    t.first_lo = (window > 0 && t.pos0 - window + 1 > 0) ? t.pos0 - window + 1 : 0;
    t.blk0 = t.first_lo / KEYS;
    t.n_iter = t.last_pos / KEYS + 1 - t.blk0;                   // key blocks [blk0, blk0 + n_iter)
    t.last_page = t.last_pos / PAGE;
    return true;
}

// The items are sorted by weight (long tiles first), so the blocks take them in a snake: pass 0 hands items
// 0 .. P-1 to blocks 0 .. P-1, pass 1 hands items P .. 2P-1 to blocks P-1 .. 0, and so on: the block with the
// heaviest item of one pass gets the lightest of the next.  (Past the end of the list the index only grows.)
__device__ __forceinline__ int snake_item(int pass, int block, int P) {
    return pass * P + ((pass & 1) ? P - 1 - block : block);
}

// Persistent: every block walks over its share of the n_work items (`snake_item`).  Barriers, tensor memory and the
// pipeline state are set up once; the counters of K/V stages and score buffers run on across items, so the first
// loads and the first S = Q K^T of the next item are under way while the softmax warps still write the
// previous item's output.  Two more barriers order the reuse of Q in shared memory (q_empty: the item's last
// S has read it) and of O in tensor memory (o_free: the softmax warps have read the finished output).
template <int DH>
__global__ void __launch_bounds__(320, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ page_table, int max_pages, int n_pages_pool,
                       GfbBatch b, int H, int G, float scale_log2e, int window, int n_x, int* status) {
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 0) { prefetch_map(&map_q); prefetch_map(&map_k); prefetch_map(&map_v); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t qs = base;                                            // [2 halves][128 rows][128 B]
    const uint32_t ks = base + TILE_BYTES;                               // KV_STAGES x same, rows = keys
    const uint32_t vs = ks + KV_STAGES * TILE_BYTES;
    Bars* bars = reinterpret_cast<Bars*>(aligned + (size_t)(1 + 2 * KV_STAGES) * TILE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rep = H / G;
    const int TQ = ROWS / rep;
    const int n_work = n_x * G;
    constexpr int NH = DH / 64;                                          // swizzled half tiles (64 dims) per operand tile

    // Rows beyond TQ * rep (heads per group that do not divide 128: 126 rows for 3, 125 for 5, ...) are never
    // written by the Q copy; they are zeroed once so that their scores are finite.  Nothing of them is stored.
    for (int i = threadIdx.x; i < (ROWS - TQ * rep) * 8 * NH; i += blockDim.x) {
        const int row = TQ * rep + i / (8 * NH), chunk = i % (8 * NH);  // NH halves x 8 chunks of 16 bytes per row
        *reinterpret_cast<uint4*>(aligned + (chunk >> 3) * HALF_BYTES + row * 128 + (chunk & 7) * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        mbar_init(smem_u32(&bars->q_empty), 1);
        mbar_init(smem_u32(&bars->o_free), 8);
        for (int s = 0; s < KV_STAGES; s++) {
            mbar_init(smem_u32(&bars->k_full[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(smem_u32(&bars->s_full[s]), 1);
            mbar_init(smem_u32(&bars->s_empty[s]), 8);
        }
        mbar_init(smem_u32(&bars->p_ready), 8);
        for (int s = 0; s < 4; s++) {
            mbar_init(smem_u32(&bars->xch[s]), 2);
            mbar_init(smem_u32(&bars->fin[s]), 2);
        }
        for (int s = 0; s < 2; s++) mbar_init(smem_u32(&bars->pv_done[s]), 1);
        mbar_init(smem_u32(&bars->o_full), 1);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    gfb_pdl_launch();
    gfb_pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t jj = 0, it = 0;                                     // key blocks and items so far
            bool ok = true;
            for (int pass = 0, w; (w = snake_item(pass, (int)blockIdx.x, (int)gridDim.x)) < n_work && ok; pass++) {
                TileWork t;
                if (!tile_work(b, w, n_x, G, TQ, window, t)) continue;
                const int* pt = page_table + (size_t)t.slot * max_pages;
                if (it > 0) ok = mbar_wait(smem_u32(&bars->q_empty), (it - 1u) & 1u, abort_flag, status, 11);
                if (!ok) break;
                // Q: rows ordered (token, head of group); a 3-D box {64 dims, rep heads, TQ tokens} per half
                mbar_expect_tx(smem_u32(&bars->q_full), (uint32_t)(NH * 128 * rep * TQ));
                tma_load_3d(qs, &map_q, 0, t.g * rep, t.t_first + t.tq0, smem_u32(&bars->q_full));
                if (NH == 2) tma_load_3d(qs + HALF_BYTES, &map_q, 64, t.g * rep, t.t_first + t.tq0, smem_u32(&bars->q_full));
                it++;
                for (int j = 0; j < t.n_iter; j++, jj++) {
                    const int s = jj % KV_STAGES;
                    const uint32_t ph = (jj / KV_STAGES) & 1u;
                    int pg[2];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        int pi = (t.blk0 + j) * 2 + h;
                        if (pi > t.last_page) pi = t.last_page;         // no such page: any finite data, masked later
                        int page = pt[pi];
                        if (page < 0 || page >= n_pages_pool) { gfb_report(status, GFB_ERR_PAGE_TABLE, t.slot, pi); page = 0; }
                        pg[h] = page;
                    }
                    if (!mbar_wait(smem_u32(&bars->s_full[s]), ph ^ 1u, abort_flag, status, 1)) { ok = false; break; }   // the scores of block jj - 2 are done
                    mbar_expect_tx(smem_u32(&bars->k_full[s]), NH * HALF_BYTES);
#pragma unroll
                    for (int h = 0; h < 2; h++) {                       // page h -> rows 64h .. 64h+63 of both halves
                        const int row = (pg[h] * G + t.g) * PAGE;
                        tma_load_2d(ks + s * TILE_BYTES + h * (PAGE * 128), &map_k, 0, row, smem_u32(&bars->k_full[s]));
                        if (NH == 2) tma_load_2d(ks + s * TILE_BYTES + HALF_BYTES + h * (PAGE * 128), &map_k, 64, row, smem_u32(&bars->k_full[s]));
                    }
                    if (!mbar_wait(smem_u32(&bars->pv_done[s]), ph ^ 1u, abort_flag, status, 2)) { ok = false; break; }   // P V of block jj - 2 is done
                    mbar_expect_tx(smem_u32(&bars->v_full[s]), NH * HALF_BYTES);
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int row = (pg[h] * G + t.g) * PAGE;
                        tma_load_2d(vs + s * TILE_BYTES + h * (PAGE * 128), &map_v, 0, row, smem_u32(&bars->v_full[s]));
                        if (NH == 2) tma_load_2d(vs + s * TILE_BYTES + HALF_BYTES + h * (PAGE * 128), &map_v, 64, row, smem_u32(&bars->v_full[s]));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(ROWS, KEYS, 0);
            constexpr uint32_t idesc_o = idesc_bf16(ROWS, DH, 1);
            uint32_t jj = 0, it = 0;
            bool ok = true;
            auto issue_s = [&](uint32_t u, bool last_of_item) -> bool {   // S of key block number u (running count)
                const int s = u % KV_STAGES, sb = u & 1u;
                if (!mbar_wait(smem_u32(&bars->k_full[s]), (u / KV_STAGES) & 1u, abort_flag, status, 3)) return false;
                if (!mbar_wait(smem_u32(&bars->s_empty[sb]), ((u >> 1) & 1u) ^ 1u, abort_flag, status, 4)) return false;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < DH / 16; k++) {
                    const uint32_t off = (k >> 2) * HALF_BYTES;
                    umma_ss(tmem + COL_S + sb * 128, desc_kmajor(qs + off) + 2 * (k & 3),
                            desc_kmajor(ks + s * TILE_BYTES + off) + 2 * (k & 3), idesc_s, k != 0);
                }
                umma_commit(smem_u32(&bars->s_full[sb]));
                if (last_of_item) umma_commit(smem_u32(&bars->q_empty));   // Q may be overwritten once these have run
                return true;
            };
            for (int pass = 0, w; (w = snake_item(pass, (int)blockIdx.x, (int)gridDim.x)) < n_work && ok; pass++) {
                TileWork t;
                if (!tile_work(b, w, n_x, G, TQ, window, t)) continue;
                ok = mbar_wait(smem_u32(&bars->q_full), it & 1u, abort_flag, status, 5);
                ok = ok && issue_s(jj, t.n_iter == 1);
                for (int j = 0; j < t.n_iter && ok; j++, jj++) {
                    if (j + 1 < t.n_iter) ok = issue_s(jj + 1, j + 2 == t.n_iter);
                    if (!ok) break;
                    const int s = jj % KV_STAGES;
                    ok = mbar_wait(smem_u32(&bars->v_full[s]), (jj / KV_STAGES) & 1u, abort_flag, status, 6);
                    ok = ok && mbar_wait(smem_u32(&bars->p_ready), jj & 1u, abort_flag, status, 7);
                    // the first P V of an item overwrites O: the previous item's output must have been read
                    if (ok && j == 0 && it > 0) ok = mbar_wait(smem_u32(&bars->o_free), (it - 1u) & 1u, abort_flag, status, 12);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 8; kk++)                       // 16 keys per MMA: 8 columns of P, 2 KB of V
                        umma_ts(tmem + COL_O, tmem + COL_P + (jj & 1u) * 64 + kk * 8,
                                desc_mnmajor(vs + s * TILE_BYTES + kk * 2048), idesc_o, (j | kk) != 0);
                    umma_commit(smem_u32(&bars->pv_done[s]));
                    if (j + 1 == t.n_iter) umma_commit(smem_u32(&bars->o_full));
                }
                it++;
            }
        }
    } else {
        // Eight softmax warps: warps 2..5 take the first 64 keys of every block, warps 6..9 the second 64.  Warp q of
        // either half holds rows 32 q .. 32 q + 31, one row per thread, so a row is shared by two warps on the same SM
        // sub-partition: while one waits for a result the other issues.  They agree on the row's maximum through
        // shared memory once per block and add their sums at the end of an item.
        const int half = warp >= 6 ? 1 : 0;
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        const int tq = r / rep;
        uint32_t jj = 0, it = 0;                                       // key blocks and items so far
        bool ok = true;
        for (int pass = 0, w; (w = snake_item(pass, (int)blockIdx.x, (int)gridDim.x)) < n_work && ok; pass++) {
            TileWork t;
            if (!tile_work(b, w, n_x, G, TQ, window, t)) continue;
            const bool row_ok = tq < t.nq;
            const int row_pos = t.pos0 + tq;
            const int row_lo = (window > 0 && row_pos - window + 1 > 0) ? row_pos - window + 1 : 0;
            float m_run = -INFINITY, l_run = 0.f;                        // l_run: this warp's half of the row's sum
            for (int j = 0; j < t.n_iter && ok; j++, jj++) {
                const uint32_t sb = jj & 1u;
                const int key0 = (t.blk0 + j) * KEYS + half * 64;        // this warp's first key
                ok = mbar_wait(smem_u32(&bars->s_full[sb]), (jj >> 1) & 1u, abort_flag, status, 8);
                if (!ok) break;
                tc_fence_after();
                const bool need_mask = key0 + 63 > t.pos0 || key0 < t.first_lo || window > 0 || t.nq < TQ;
                // this warp's half of the row into registers
                uint32_t raw[2][32];
                tmem_ld32_issue(lane_base + COL_S + sb * 128 + half * 64, raw[0]);
                tmem_ld32_issue(lane_base + COL_S + sb * 128 + half * 64 + 32, raw[1]);
                tmem_ld_wait32(raw[0]);
                tmem_ld_wait32(raw[1]);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->s_empty[sb]));    // one arrival per warp
                float v[2][32];
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) v[c][i] = __uint_as_float(raw[c][i]);
                if (need_mask) {                                             // only blocks on the diagonal or at the window's edge
#pragma unroll
                    for (int c = 0; c < 2; c++)
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int kj = key0 + c * 32 + i;
                            if (!(row_ok && kj <= row_pos && kj >= row_lo)) v[c][i] = -INFINITY;
                        }
                }
                float mx4[4];                                                // four chains
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const float* x = &v[c >> 1][(c & 1) * 16];
                    mx4[c] = fmaxf(x[0], x[1]);
#pragma unroll
                    for (int i = 2; i < 16; i += 2) mx4[c] = max3(mx4[c], x[i], x[i + 1]);
                }
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // the other half's maximum (buffers by block parity: a warp cannot be two blocks ahead of its partner)
                bars->mx_half[sb][half][r] = mx;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->xch[q]));
                ok = mbar_wait(smem_u32(&bars->xch[q]), jj & 1u, abort_flag, status, 13);
                if (!ok) break;
                mx = fmaxf(mx, bars->mx_half[sb][half ^ 1][r]);
                // The running maximum only has to keep the exponentials in range, so it follows the true maximum
                // lazily: it moves (and O is rescaled) only when the true maximum has grown by more than 2^8 in
                // the exponent; until then probabilities may reach 256, which bfloat16 and the 32-bit sums hold.
                // Sum and output use the same reference, so the quotient at the end is exact either way.
                float m_new = m_run;
                if (mx > m_run && (m_run == -INFINITY || (mx - m_run) * scale_log2e > 8.f)) m_new = mx;
                const float corr = (m_run == -INFINITY || m_new == m_run) ? 1.f : fast_exp2((m_run - m_new) * scale_log2e);   // a row without keys so far has O = 0, l = 0
                const float mneg = (m_new == -INFINITY) ? 0.f : -m_new * scale_log2e;
                // probabilities (2^-inf = 0 for masked scores), rounded to bfloat16 into tensor memory
                float rs2[2] = {0.f, 0.f};
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t pk[16];
                    float rs_odd = 0.f;                                      // rs2[c] and rs_odd: one packed sum
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float t0, t1;
                        fma2(v[c][i], v[c][i + 1], scale_log2e, mneg, t0, t1);
                        const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                        add2(rs2[c], rs_odd, p0, p1);
                        pk[i >> 1] = pack2(p0, p1);
                    }
                    rs2[c] += rs_odd;
                    tmem_st16(lane_base + COL_P + sb * 64 + half * 32 + c * 16, pk);
                }
                const float rs = rs2[0] + rs2[1];
                // O of the earlier blocks follows the new maximum, each warp its 64 columns, after the previous P V has
                // landed.  Rarely, so most phases of that barrier are never looked at; the parity wait is valid all the
                // same: the phase before the awaited one (P V of block jj - 3) is over, since the scores of this block
                // were issued behind the P V of block jj - 2, and the phase after it (block jj + 1) cannot have begun,
                // since that P V is issued behind this block's, which waits for this warp's arrival below.
                if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                    ok = mbar_wait(smem_u32(&bars->pv_done[(jj - 1u) & 1u]), ((jj - 1u) >> 1) & 1u, abort_flag, status, 9);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < NH; c++) {
                        float o[32];
                        tmem_ld32(lane_base + COL_O + half * (DH / 2) + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] *= corr;
                        tmem_st32(lane_base + COL_O + half * (DH / 2) + c * 32, o);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->p_ready));
                l_run = l_run * corr + rs;
                m_run = m_new;
            }
            // All P V of the item have landed: a barrier of its own with one phase per item.  (A parity wait on pv_done
            // is only valid while that barrier can be neither a phase behind nor a phase ahead of the awaited one; at the
            // end of an item, with the waits of the earlier blocks left out, it could be either.)
            if (ok) ok = mbar_wait(smem_u32(&bars->o_full), it & 1u, abort_flag, status, 10);
            if (!ok) break;
            tc_fence_after();
            // the row's sum: both halves are under the same reference
            bars->l_half[it & 1u][half][r] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->fin[q]));
            ok = mbar_wait(smem_u32(&bars->fin[q]), it & 1u, abort_flag, status, 14);
            if (!ok) break;
            l_run += bars->l_half[it & 1u][half ^ 1][r];
            it++;
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const int head = t.g * rep + (r - tq * rep);
            __nv_bfloat16* dst = out + ((size_t)(t.t_first + t.tq0 + tq) * H + head) * DH + half * (DH / 2);   // each warp stores its half of the columns
#pragma unroll 1
            for (int c = 0; c < NH; c++) {
                float v[32];
                tmem_ld32(lane_base + COL_O + half * (DH / 2) + c * 32, v);   // warp-collective: also for idle rows
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pk;
                        pk.x = pack2(v[i] * inv, v[i + 1] * inv); pk.y = pack2(v[i + 2] * inv, v[i + 3] * inv);
                        pk.z = pack2(v[i + 4] * inv, v[i + 5] * inv); pk.w = pack2(v[i + 6] * inv, v[i + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->o_free));         // O may be overwritten by the next item
        }
    }

    if (*abort_flag) {
        unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 50000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---- two query tiles per block ------------------------------------------------------------------
// The same algorithm with TWO tiles of 128 rows (2 TQ consecutive tokens) in one block, each with its own
// four softmax warps, sharing every K/V page that is loaded.  The tensor pipe alternates between the
// tiles: while the warps of one tile work through their exponentials, it computes P V of the other tile
// and that tile's next scores.  Tensor memory: S of tile x in columns 128 x .. 128 x + 127, O of tile x in
// 256 + 128 x ...; P (bfloat16) overwrites the first 64 columns of its own S once the scores are in
// registers, and the next S of that tile is issued behind the P V that reads it (the pipe runs in order).
struct Bars2 {
    unsigned long long q_full;
    unsigned long long k_full[KV_STAGES], k_empty[KV_STAGES];
    unsigned long long v_full[KV_STAGES], v_empty[KV_STAGES];
    unsigned long long s_full[2];
    unsigned long long p_ready[2];
    unsigned long long pv_done[2];
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void __launch_bounds__(320, 1)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ page_table, int max_pages, int n_pages_pool,
                        GfbBatch b, int H, int G, float scale_log2e, int window, int* status) {
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 0) { prefetch_map(&map_q); prefetch_map(&map_k); prefetch_map(&map_v); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t qs = base;                                            // 2 tiles x [2 halves][128 rows][128 B]
    const uint32_t ks = base + 2 * TILE_BYTES;
    const uint32_t vs = ks + KV_STAGES * TILE_BYTES;
    Bars2* bars = reinterpret_cast<Bars2*>(aligned + (size_t)(2 + 2 * KV_STAGES) * TILE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rep = H / G;
    const int TQ = ROWS / rep;
    for (int i = threadIdx.x; i < 2 * (ROWS - TQ * rep) * 16; i += blockDim.x) {      // both tiles' idle rows, as in the one-tile kernel
        const int x = i / ((ROWS - TQ * rep) * 16), k = i - x * (ROWS - TQ * rep) * 16;
        const int row = TQ * rep + (k >> 4), chunk = k & 15;
        *reinterpret_cast<uint4*>(aligned + x * TILE_BYTES + (chunk >> 3) * HALF_BYTES + row * 128 + (chunk & 7) * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    int seq = -1, tq0 = 0;
    {
        int left = (int)gridDim.x - 1 - (int)blockIdx.x;                 // long tiles first
        for (int i = 0; i < b.n_seqs; i++) {
            int qlen = b.cu_seqlens[i + 1] - b.cu_seqlens[i];
            int nt = (qlen + 2 * TQ - 1) / (2 * TQ);
            if (left < nt) { seq = i; tq0 = left * 2 * TQ; break; }
            left -= nt;
        }
    }
    if (seq < 0) return;
    const int g = blockIdx.y;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        for (int s = 0; s < KV_STAGES; s++) {
            mbar_init(smem_u32(&bars->k_full[s]), 1);
            mbar_init(smem_u32(&bars->k_empty[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        for (int x = 0; x < 2; x++) {
            mbar_init(smem_u32(&bars->s_full[x]), 1);
            mbar_init(smem_u32(&bars->p_ready[x]), 4);
            mbar_init(smem_u32(&bars->pv_done[x]), 1);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    gfb_pdl_launch();
    gfb_pdl_wait();

    const int t_first = b.cu_seqlens[seq];
    const int qlen = b.cu_seqlens[seq + 1] - t_first;
    const int slot = b.slots[seq];
    const int len0 = b.lengths[slot];
    // per tile: tokens [tq0 + x TQ, +nq), positions from pos0, key blocks [lo_blk, hi_blk)
    int nq[2], pos0[2], lo_blk[2], hi_blk[2];
#pragma unroll
    for (int x = 0; x < 2; x++) {
        nq[x] = min(TQ, qlen - (tq0 + x * TQ));
        pos0[x] = len0 + tq0 + x * TQ;
        if (nq[x] > 0) {
            const int first_lo = (window > 0 && pos0[x] - window + 1 > 0) ? pos0[x] - window + 1 : 0;
            lo_blk[x] = first_lo / KEYS;
            hi_blk[x] = (pos0[x] + nq[x] - 1) / KEYS + 1;
        } else {
            lo_blk[x] = 0;
            hi_blk[x] = 0;
        }
    }
    const int blk0 = nq[1] > 0 ? min(lo_blk[0], lo_blk[1]) : lo_blk[0];
    const int blk1 = max(hi_blk[0], hi_blk[1]);
    const int n_iter = blk1 - blk0;
    const int last_page = (len0 + min(qlen, tq0 + 2 * TQ) - 1) / PAGE;
    const int* pt = page_table + (size_t)slot * max_pages;
    auto active = [&](int x, int j) { return blk0 + j >= lo_blk[x] && blk0 + j < hi_blk[x]; };

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&bars->q_full), (uint32_t)(2 * 2 * 128 * rep * TQ));
#pragma unroll
            for (int x = 0; x < 2; x++) {                                // rows beyond the batch are filled with zeros
                tma_load_3d(qs + x * TILE_BYTES, &map_q, 0, g * rep, t_first + tq0 + x * TQ, smem_u32(&bars->q_full));
                tma_load_3d(qs + x * TILE_BYTES + HALF_BYTES, &map_q, 64, g * rep, t_first + tq0 + x * TQ, smem_u32(&bars->q_full));
            }
            for (int j = 0; j < n_iter; j++) {
                const int s = j % KV_STAGES;
                const uint32_t ph = (uint32_t)(j / KV_STAGES) & 1u;
                int pg[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    int pi = (blk0 + j) * 2 + h;
                    if (pi > last_page) pi = last_page;
                    int page = pt[pi];
                    if (page < 0 || page >= n_pages_pool) { gfb_report(status, GFB_ERR_PAGE_TABLE, slot, pi); page = 0; }
                    pg[h] = page;
                }
                if (!mbar_wait(smem_u32(&bars->k_empty[s]), ph ^ 1u, abort_flag, status, 1)) break;
                mbar_expect_tx(smem_u32(&bars->k_full[s]), TILE_BYTES);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int row = (pg[h] * G + g) * PAGE;
                    tma_load_2d(ks + s * TILE_BYTES + h * (PAGE * 128), &map_k, 0, row, smem_u32(&bars->k_full[s]));
                    tma_load_2d(ks + s * TILE_BYTES + HALF_BYTES + h * (PAGE * 128), &map_k, 64, row, smem_u32(&bars->k_full[s]));
                }
                if (!mbar_wait(smem_u32(&bars->v_empty[s]), ph ^ 1u, abort_flag, status, 2)) break;
                mbar_expect_tx(smem_u32(&bars->v_full[s]), TILE_BYTES);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int row = (pg[h] * G + g) * PAGE;
                    tma_load_2d(vs + s * TILE_BYTES + h * (PAGE * 128), &map_v, 0, row, smem_u32(&bars->v_full[s]));
                    tma_load_2d(vs + s * TILE_BYTES + HALF_BYTES + h * (PAGE * 128), &map_v, 64, row, smem_u32(&bars->v_full[s]));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(ROWS, KEYS, 0);
            constexpr uint32_t idesc_o = idesc_bf16(ROWS, D, 1);
            uint32_t n_pv[2] = {0, 0};                                   // P V products issued per tile
            bool ok = mbar_wait(smem_u32(&bars->q_full), 0, abort_flag, status, 5);
            auto issue_s = [&](int x, int j) {                           // K stage of block j is known to be loaded
                const int s = j % KV_STAGES;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const uint32_t off = (k >> 2) * HALF_BYTES;
                    umma_ss(tmem + 128 * x, desc_kmajor(qs + x * TILE_BYTES + off) + 2 * (k & 3),
                            desc_kmajor(ks + s * TILE_BYTES + off) + 2 * (k & 3), idesc_s, k != 0);
                }
                umma_commit(smem_u32(&bars->s_full[x]));
            };
            auto k_ready = [&](int j) {
                return mbar_wait(smem_u32(&bars->k_full[j % KV_STAGES]), (uint32_t)(j / KV_STAGES) & 1u, abort_flag, status, 3);
            };
            if (ok && n_iter > 0) {
                ok = k_ready(0);
                if (ok) {
                    tc_fence_after();
                    if (active(0, 0)) issue_s(0, 0);
                    if (active(1, 0)) issue_s(1, 0);
                    umma_commit(smem_u32(&bars->k_empty[0]));
                }
            }
            for (int j = 0; j < n_iter && ok; j++) {
                const int s = j % KV_STAGES;
                bool k_next = false;                                     // whether K of block j + 1 has been waited for
                ok = mbar_wait(smem_u32(&bars->v_full[s]), (uint32_t)(j / KV_STAGES) & 1u, abort_flag, status, 6);
#pragma unroll
                for (int x = 0; x < 2 && ok; x++) {
                    if (active(x, j)) {
                        ok = mbar_wait(smem_u32(&bars->p_ready[x]), n_pv[x] & 1u, abort_flag, status, 7);
                        if (!ok) break;
                        tc_fence_after();
#pragma unroll
                        for (int kk = 0; kk < 8; kk++)                   // 16 keys per MMA: 8 columns of P, 2 KB of V
                            umma_ts(tmem + 256 + 128 * x, tmem + 128 * x + kk * 8,
                                    desc_mnmajor(vs + s * TILE_BYTES + kk * 2048), idesc_o, (n_pv[x] | (uint32_t)kk) != 0);
                        umma_commit(smem_u32(&bars->pv_done[x]));
                        n_pv[x]++;
                    }
                    if (j + 1 < n_iter && active(x, j + 1)) {            // the tile's next scores, behind its P V
                        if (!k_next) { ok = k_ready(j + 1); k_next = true; if (!ok) break; tc_fence_after(); }
                        issue_s(x, j + 1);
                    }
                }
                if (!ok) break;
                umma_commit(smem_u32(&bars->v_empty[s]));
                if (j + 1 < n_iter) {
                    if (!k_next) { ok = k_ready(j + 1); if (!ok) break; }
                    umma_commit(smem_u32(&bars->k_empty[(j + 1) % KV_STAGES]));
                }
            }
        }
    } else {
        const int x = (warp - 2) >> 2;                                   // warps 2..5: tile 0, warps 6..9: tile 1
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
        const uint32_t col_s = 128 * x, col_o = 256 + 128 * x;
        const int tq = r / rep;
        const bool row_ok = tq < nq[x];
        const int row_pos = pos0[x] + tq;
        const int row_lo = (window > 0 && row_pos - window + 1 > 0) ? row_pos - window + 1 : 0;
        const int first_lo = (window > 0 && pos0[x] - window + 1 > 0) ? pos0[x] - window + 1 : 0;
        float m_run = -INFINITY, l_run = 0.f;
        uint32_t n_done = 0;                                             // blocks of this tile finished
        bool ok = true;
        for (int j = 0; j < n_iter && ok; j++) {
            if (!active(x, j)) continue;
            const int key0 = (blk0 + j) * KEYS;
            ok = mbar_wait(smem_u32(&bars->s_full[x]), n_done & 1u, abort_flag, status, 8);
            if (!ok) break;
            tc_fence_after();
            const bool need_mask = key0 + KEYS - 1 > pos0[x] || key0 < first_lo || window > 0 || nq[x] < TQ;
            float v[4][32];
            tmem_ld_row128(lane_base + col_s, v);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 4; c++)
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        const int kj = key0 + c * 32 + i;
                        if (!(row_ok && kj <= row_pos && kj >= row_lo)) v[c][i] = -INFINITY;
                    }
            }
            float mx4[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                mx4[c] = fmaxf(v[c][0], v[c][1]);
#pragma unroll
                for (int i = 2; i < 32; i += 2) mx4[c] = max3(mx4[c], v[c][i], v[c][i + 1]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float m_new = m_run;                                         // lazy reference maximum, as in the one-tile kernel
            if (mx > m_run && (m_run == -INFINITY || (mx - m_run) * scale_log2e > 8.f)) m_new = mx;
            const float corr = (m_run == -INFINITY || m_new == m_run) ? 1.f : fast_exp2((m_run - m_new) * scale_log2e);   // a row without keys so far has O = 0, l = 0
            const float mneg = (m_new == -INFINITY) ? 0.f : -m_new * scale_log2e;
            // P over the first half of this tile's own scores: all of this row's scores are in registers by now,
            // and a thread only ever touches its own row (lane) of tensor memory
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t pk[16];
                float rs_odd = 0.f;                                      // rs4[c] and rs_odd: one packed sum
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float t0, t1;
                    fma2(v[c][i], v[c][i + 1], scale_log2e, mneg, t0, t1);
                    const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                    add2(rs4[c], rs_odd, p0, p1);
                    pk[i >> 1] = pack2(p0, p1);
                }
                rs4[c] += rs_odd;
                tmem_st16(lane_base + col_s + c * 16, pk);
            }
            // O follows the reference maximum, rarely (S of this block was issued behind the tile's previous P V, so
            // that phase is over and the wait only orders the accesses)
            if (n_done > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                ok = mbar_wait(smem_u32(&bars->pv_done[x]), (n_done - 1u) & 1u, abort_flag, status, 9);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    float o[32];
                    tmem_ld32(lane_base + col_o + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] *= corr;
                    tmem_st32(lane_base + col_o + c * 32, o);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->p_ready[x]));
            l_run = l_run * corr + (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            m_run = m_new;
            n_done++;
        }
        if (ok && n_done > 0) ok = mbar_wait(smem_u32(&bars->pv_done[x]), (n_done - 1u) & 1u, abort_flag, status, 10);
        if (ok && n_done > 0) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const int head = g * rep + (r - tq * rep);
            __nv_bfloat16* dst = out + ((size_t)(t_first + tq0 + x * TQ + tq) * H + head) * D;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                float v[32];
                tmem_ld32(lane_base + col_o + c * 32, v);
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 pk;
                        pk.x = pack2(v[i] * inv, v[i + 1] * inv); pk.y = pack2(v[i + 2] * inv, v[i + 3] * inv);
                        pk.z = pack2(v[i + 4] * inv, v[i + 5] * inv); pk.w = pack2(v[i + 6] * inv, v[i + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
                    }
                }
            }
        }
    }

    if (*abort_flag) {
        unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 50000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
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

}  // namespace

// Causal attention for runs of new tokens on tcgen05; head_dim 128, pages of 64, at most 8 heads per group
// with 128 % (heads per group) == 0.  tiles: query tiles of 128 rows per block, 1 or 2, or 0 to let the
// function choose by the amount of work.  max_blocks: cap of the one-tile kernel's grid (0: one block per SM).
GFB_API int gfb_attn_prefill_tc(const void* q, void* out, void* k_pool, void* v_pool, const int* page_table, int max_pages,
                                int page_size, int n_pages, const int* cu_seqlens, const int* tok_seq, const int* slots,
                                const int* lengths, int n_seqs, int n_tokens, int H, int G, int d, float scale, int window,
                                int tiles, int max_blocks, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (page_size != PAGE || (d != 64 && d != 128))
        return gfb_fail("gfb_attn_prefill_tc: built for pages of %d and head_dim 64 or 128, got %d and %d", PAGE, page_size, d);
    if (G <= 0 || H % G) return gfb_fail("gfb_attn_prefill_tc: %d heads over %d groups", H, G);
    const int rep = H / G;
    if (rep > 8) return gfb_fail("gfb_attn_prefill_tc: %d heads per group (at most 8)", rep);
    const int TQ = ROWS / rep;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return gfb_fail("gfb_attn_prefill_tc: the driver does not export cuTensorMapEncodeTiled");
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)H, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)H * d * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)rep, (cuuint32_t)TQ};
        cuuint32_t es[3] = {1, 1, 1};
        CUresult r = enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return gfb_fail("gfb_attn_prefill_tc: tensor map of q refused (%d)", (int)r);
    }
    if ((long long)n_pages * G * PAGE > 2147483647LL)           // TMA coordinates are 32-bit
        return gfb_fail("gfb_attn_prefill_tc: %d pages x %d heads x %d tokens do not fit the 32-bit row coordinate of a tensor map",
                        n_pages, G, PAGE);
    for (int i = 0; i < 2; i++) {
        cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)n_pages * G * PAGE};
        cuuint64_t strides[1] = {(cuuint64_t)d * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)PAGE};
        cuuint32_t es[2] = {1, 1};
        CUresult r = enc(i ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, i ? v_pool : k_pool, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return gfb_fail("gfb_attn_prefill_tc: tensor map of the cache refused (%d)", (int)r);
    }
    GfbBatch b{cu_seqlens, tok_seq, slots, lengths, n_seqs, n_tokens};
    if (tiles < 0 || tiles > 2) return gfb_fail("gfb_attn_prefill_tc: %d query tiles per block (0 = choose, 1 or 2)", tiles);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    }
    cudaError_t e;
    const long blocks2 = ((long)(n_tokens + 2 * TQ - 1) / (2 * TQ)) * G;
    if (d == 128 && (tiles == 2 || (tiles == 0 && blocks2 >= 6L * sms))) {
        // enough work for several rounds of blocks of two tiles, which share their K/V loads and keep the tensor
        // pipe busier (measured: from about 7,000 tokens of one sequence on, at 32 heads in 8 groups); with less
        // work the persistent one-tile kernel balances the SMs better
        size_t smem = 1024 + (size_t)(2 + 2 * KV_STAGES) * TILE_BYTES + sizeof(Bars2);
        static size_t configured2 = 0;
        if (smem > configured2) {
            cudaError_t a = cudaFuncSetAttribute(attn_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (a != cudaSuccess) return gfb_fail("gfb_attn_prefill_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(a));
            configured2 = smem;
        }
        dim3 grid((n_tokens + 2 * TQ - 1) / (2 * TQ) + n_seqs, G);
        e = gfb_launch(attn_prefill_tc2_kernel, grid, dim3(320), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                       page_table, max_pages, n_pages, b, H, G, scale * 1.4426950408889634f, window, status);
    } else {
        size_t smem = 1024 + (size_t)(1 + 2 * KV_STAGES) * TILE_BYTES + sizeof(Bars);
        static bool configured = false;
        if (!configured) {
            cudaError_t a = cudaFuncSetAttribute(attn_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (a == cudaSuccess) a = cudaFuncSetAttribute(attn_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (a != cudaSuccess) return gfb_fail("gfb_attn_prefill_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(a));
            configured = true;
        }
        const int n_x = (n_tokens + TQ - 1) / TQ + n_seqs;           // an upper bound of the tiles; surplus items are empty
        long blocks = (long)n_x * G;
        const long cap = max_blocks > 0 ? max_blocks : sms;           // one block per SM walks over the items
        if (blocks > cap) blocks = cap;
        if (d == 128)
            e = gfb_launch(attn_prefill_tc_kernel<128>, dim3((unsigned)blocks), dim3(320), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                           page_table, max_pages, n_pages, b, H, G, scale * 1.4426950408889634f, window, n_x, status);
        else
            e = gfb_launch(attn_prefill_tc_kernel<64>, dim3((unsigned)blocks), dim3(320), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                           page_table, max_pages, n_pages, b, H, G, scale * 1.4426950408889634f, window, n_x, status);
    }
    return gfb_check(e, "gfb_attn_prefill_tc");
}

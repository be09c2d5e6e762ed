// bfloat16 matrix products on the 5th-generation tensor cores of sm_100a:
// operands staged in shared memory by TMA (128-byte swizzle), tcgen05.mma issued
// by one thread, the 32-bit accumulator in tensor memory, read back with
// tcgen05.ld for a fused epilogue.
//
// It computes D[r, c] = sum_k X[r, k] * Y[c, k] for two K-major operands, which
// is how both the activations [M, K] and nn.Linear's weights [N, K] lie in
// memory (gpt-fast model.py:174-175, :222-224).  X supplies the 128 rows of the
// MMA, Y its N columns:
//   normal  (prefill, many tokens): X = activations, Y = weights, tile 128 x BN
//   swapped (decode, few tokens):   X = weights, Y = activations; the 128 MMA
//            rows are weight rows, the tokens (padded to 16..128) are the MMA
//            columns, so a step streams each weight byte once at full width.
// Epilogues: store (bf16 or f32), add into the 32-bit residual, SwiGLU over
// weight rows that alternate gate/up, or (swapped only) a 32-bit partial for a
// split over K that `splitk_reduce_kernel` sums in a fixed order.
//
// Roles in a block of 192 threads: warp 0 = TMA producer (one lane), warp 1 =
// tensor-memory allocation + MMA issue (one lane), warps 2..5 = epilogue (one
// quarter of the 128 accumulator lanes each).  Stages of the shared-memory ring
// are handed over through mbarriers.  Every wait is bounded by wall-clock time:
// when one runs out the block records GFB_ERR_WAIT_TIMEOUT in `status`, lets
// copies in flight land, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

GFB_DEFINE_LAST_ERROR()

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

namespace {

constexpr int BM = 128;              // MMA rows per tile
constexpr int BK = 64;               // k per stage: 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;           // k of one tcgen05.mma for 16-bit inputs
constexpr int MAX_STAGES = 12;
constexpr int X_TILE_BYTES = BM * BK * 2;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;    // 2 s: far beyond any healthy wait

struct Barriers {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long accum;
    uint32_t tmem_base;
    int abort_flag;
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
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Wait for the phase with `parity` to complete; false when the block aborts or time runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int which) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 128; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            gfb_report(status, GFB_ERR_WAIT_TIMEOUT, which, (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)));
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

// The same with an L2 policy: weights of a decode step are read once per step and are far larger than L2, so they
// are marked to be evicted first and leave the cache to what is read again soon (activations, partial sums, the
// key/value pages).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);      // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// The columns of an epilogue round with one instruction and one wait (four loads of sixteen in flight together made
// the compiler spill).
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {"
        "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16_raw(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32_raw(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {"
        "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
template <int N> __device__ __forceinline__ void tmem_ld_group(uint32_t taddr, uint32_t (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld_group<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16_raw(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_group<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32_raw(taddr, r); }
template <> __device__ __forceinline__ void tmem_ld_group<64>(uint32_t taddr, uint32_t (&r)[64]) { tmem_ld64(taddr, r); }

// Barrier number 1 for the four epilogue warps (128 threads), alone or with the AND of a flag over them.
__device__ __forceinline__ void epilogue_warps_sync() { asm volatile("barrier.cta.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool epilogue_warps_all(bool flag) {
    uint32_t all;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(all) : "r"((uint32_t)flag) : "memory");
    return all != 0;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- epilogue of the normal orientation -------------------------------------------------
// The accumulator has one row (token) per thread, which would make every global access a
// 32-row gather.  So each epilogue warp first copies its 32 accumulator rows from tensor memory
// to shared memory (the ring is free by then; rows padded by 4 floats so the copies do not
// collide on banks), then walks ITS rows with all lanes side by side along a row: global reads
// and writes are whole contiguous lines, and the residual loads of four rows are in flight
// together.  Only __syncwarp is needed: a warp reads back what it wrote itself.
template <int BN, int EPI, typename TO>
__device__ __forceinline__ void epilogue_rows(float* stage, uint32_t taddr, int q, int lane, TO* out, int row0, int col0,
                                              int R, int N, int ldo) {
    constexpr int SP = BN + 4;
    float* mine = stage + (size_t)(q * 32 + lane) * SP;
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
        float v[16];
        tmem_ld16(taddr + c, v);
#pragma unroll
        for (int j = 0; j < 16; j += 4) *reinterpret_cast<float4*>(mine + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    __syncwarp();
    const int rows = min(32, R - (row0 + q * 32));
    if (EPI == EPI_ADD) {
        constexpr int PASSES = BN >= 128 ? BN / 128 : 1;        // 32 lanes x float4 = 128 columns per pass
#pragma unroll 1
        for (int rr = 0; rr < rows; rr += 4) {
            float4 res[4][PASSES];
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    int col = col0 + ps * 128 + lane * 4;
                    if (rr + u < rows && col < N)
                        res[u][ps] = *reinterpret_cast<const float4*>((float*)out + (size_t)(row0 + q * 32 + rr + u) * ldo + col);
                }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int ps = 0; ps < PASSES; ps++) {
                    int col = col0 + ps * 128 + lane * 4;
                    if (rr + u < rows && col < N) {
                        float4 a = *reinterpret_cast<const float4*>(stage + (size_t)(q * 32 + rr + u) * SP + ps * 128 + lane * 4);
                        float4 x = res[u][ps];
                        x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w;
                        *reinterpret_cast<float4*>((float*)out + (size_t)(row0 + q * 32 + rr + u) * ldo + col) = x;
                    }
                }
        }
    } else if (EPI == EPI_SWIGLU) {
        // 8 accumulator columns (4 gate/up pairs) per lane -> 4 outputs
#pragma unroll 2
        for (int rr = 0; rr < rows; rr++) {
            int c = lane * 8;
            if (c < BN && col0 + c < N) {
                const float* a = stage + (size_t)(q * 32 + rr) * SP + c;
                float4 lo = *reinterpret_cast<const float4*>(a), hi = *reinterpret_cast<const float4*>(a + 4);
                uint2 pk;
                pk.x = pack_bf16(silu_mul(lo.x, lo.y), silu_mul(lo.z, lo.w));
                pk.y = pack_bf16(silu_mul(hi.x, hi.y), silu_mul(hi.z, hi.w));
                *reinterpret_cast<uint2*>((__nv_bfloat16*)out + (size_t)(row0 + q * 32 + rr) * ldo + ((col0 + c) >> 1)) = pk;
            }
        }
    } else if (sizeof(TO) == 4) {
        constexpr int PASSES = BN >= 128 ? BN / 128 : 1;
#pragma unroll 2
        for (int rr = 0; rr < rows; rr++)
#pragma unroll
            for (int ps = 0; ps < PASSES; ps++) {
                int c = ps * 128 + lane * 4;
                if (col0 + c < N)
                    *reinterpret_cast<float4*>((float*)out + (size_t)(row0 + q * 32 + rr) * ldo + col0 + c) =
                        *reinterpret_cast<const float4*>(stage + (size_t)(q * 32 + rr) * SP + c);
            }
    } else {
#pragma unroll 2
        for (int rr = 0; rr < rows; rr++) {
            int c = lane * 8;
            if (c < BN && col0 + c < N) {
                const float* a = stage + (size_t)(q * 32 + rr) * SP + c;
                float4 lo = *reinterpret_cast<const float4*>(a), hi = *reinterpret_cast<const float4*>(a + 4);
                uint4 pk;
                pk.x = pack_bf16(lo.x, lo.y); pk.y = pack_bf16(lo.z, lo.w);
                pk.z = pack_bf16(hi.x, hi.y); pk.w = pack_bf16(hi.z, hi.w);
                *reinterpret_cast<uint4*>((__nv_bfloat16*)out + (size_t)(row0 + q * 32 + rr) * ldo + col0 + c) = pk;
            }
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------
// X: [R, K] rows of the MMA; Y: [Cc, K] columns of the MMA.  SWAP = false: rows are
// tokens, out[r * ldo + c]; SWAP = true: rows are weight rows, out[c * ldo + r].
template <int BN, bool SWAP, int EPI, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
               TO* __restrict__ out, float* __restrict__ partial, int R, int Cc, int K, int ldo,
               int kb_per_split, int stages, int* status) {
    constexpr int Y_TILE_BYTES = BN * BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 32) { prefetch_map(&map_x); prefetch_map(&map_y); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t xs = base;
    const uint32_t ys = base + (uint32_t)stages * X_TILE_BYTES;
    Barriers* bars = reinterpret_cast<Barriers*>(aligned + (size_t)stages * (X_TILE_BYTES + Y_TILE_BYTES));
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * BM, col0 = blockIdx.y * BN;
    const int total_kb = (K + BK - 1) / BK;
    const int kb0 = blockIdx.z * kb_per_split;
    const int nkb = min(kb_per_split, total_kb - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        mbar_init(smem_u32(&bars->accum), 1);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // Weights are written by no kernel: the ring is filled with weight tiles at once, before the block's tensor
        // memory is there and before the wait for the previous kernel (no other thread touches the barriers before
        // the block's barrier below).
        const int n_pre = min(stages, nkb);
        for (int i = 0; i < n_pre; i++) {                   // fresh barriers: every stage is free
            uint32_t full = smem_u32(&bars->full[i]);
            mbar_expect_tx(full, X_TILE_BYTES + Y_TILE_BYTES);
            if (SWAP) tma_load_2d_hint(xs + i * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full, l2_evict_first_policy());
            else tma_load_2d(ys + i * Y_TILE_BYTES, &map_y, (kb0 + i) * BK, col0, full);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    // This block now holds everything it needs (shared memory, tensor memory): the next kernel
    // in the stream may become resident.  Weights are written by no kernel, so the producer
    // fills the ring with weight tiles before it waits for the previous kernel; everything
    // else (activations, the residual, the partials) is touched only after the wait.
    gfb_pdl_launch();
    if (!(warp == 0 && lane == 0)) gfb_pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            const int n_pre = min(stages, nkb);             // their weight halves are on their way already
            const uint64_t pol = l2_evict_first_policy();
            gfb_pdl_wait();
            for (int i = 0; i < n_pre; i++) {
                uint32_t full = smem_u32(&bars->full[i]);
                if (SWAP) tma_load_2d(ys + i * Y_TILE_BYTES, &map_y, (kb0 + i) * BK, col0, full);
                else tma_load_2d(xs + i * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full);
            }
            for (int i = n_pre; i < nkb; i++) {
                int s = i % stages;
                uint32_t ph = (uint32_t)(i / stages) & 1u;
                if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag, status, 1)) break;
                uint32_t full = smem_u32(&bars->full[s]);
                mbar_expect_tx(full, X_TILE_BYTES + Y_TILE_BYTES);
                if (SWAP) tma_load_2d_hint(xs + s * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full, pol);
                else tma_load_2d(xs + s * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full);
                tma_load_2d(ys + s * Y_TILE_BYTES, &map_y, (kb0 + i) * BK, col0, full);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            for (int i = 0; i < nkb && ok; i++) {
                int s = i % stages;
                uint32_t ph = (uint32_t)(i / stages) & 1u;
                ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag, status, 2);
                if (!ok) break;
                tc_fence_after();
                uint64_t da = umma_smem_desc(xs + s * X_TILE_BYTES);
                uint64_t db = umma_smem_desc(ys + s * Y_TILE_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; k++)       // 32 bytes further along K: +2 in 16-byte units
                    umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
                umma_commit(smem_u32(&bars->empty[s]));    // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(smem_u32(&bars->accum));
        }
    } else {
        const int q = warp & 3;                             // tensor-memory lanes 32q .. 32q+31 belong to this warp
        const int r = row0 + q * 32 + lane;
        bool ok = mbar_wait(smem_u32(&bars->accum), 0, abort_flag, status, 3);
        tc_fence_after();
        {
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
            if constexpr (!SWAP) {
                if (ok && row0 + q * 32 < R)
                    epilogue_rows<BN, EPI == EPI_PARTIAL ? EPI_STORE : EPI, TO>(reinterpret_cast<float*>(aligned), taddr, q, lane,
                                                                                out, row0, col0, R, Cc, ldo);
            } else {
            // Up to 64 accumulator columns (tokens) a round, brought from tensor memory by one load.
            constexpr int GROUP = BN < 64 ? BN : 64;
            // From 32 tokens on the tile goes through shared memory (the ring is free by now): a thread owns one weight
            // row, so its direct stores are 4 bytes each, 128 per warp and token, and 64 of them per thread kept a
            // block for 3 us; from the staged tile a warp writes a token's 128 rows with one 16-byte store per lane.
            const int ldv = EPI == EPI_PARTIAL ? R : ldo;
            const bool staged = BN >= 32 && R % 4 == 0 && ldv % (EPI == EPI_SWIGLU ? 2 : 4) == 0;   // uniform over the grid
            if (staged) {
                float* tile = reinterpret_cast<float*>(aligned);        // [tokens][128 rows]
                const bool all_ok = epilogue_warps_all(ok);             // all four warps or none
                if (all_ok) {
#pragma unroll 1
                    for (int c = 0; c < BN; c += GROUP) {
                        if (col0 + c >= Cc) break;                      // uniform: nothing left in this tile
                        uint32_t raw[GROUP];
                        tmem_ld_group<GROUP>(taddr + c, raw);
#pragma unroll
                        for (int j = 0; j < GROUP; j++) tile[(c + j) * BM + q * 32 + lane] = __uint_as_float(raw[j]);
                    }
                    epilogue_warps_sync();
                    const int n_tok = min(BN, Cc - col0);
                    const int rr = row0 + 4 * lane;                     // this lane's four rows of every token
#pragma unroll 2
                    for (int j = q; j < n_tok; j += 4) {
                        const int m = col0 + j;
                        const float4 v = *reinterpret_cast<const float4*>(tile + j * BM + 4 * lane);
                        const float e[4] = {v.x, v.y, v.z, v.w};
                        if (rr + 3 < R) {
                            if (EPI == EPI_SWIGLU) {
                                *reinterpret_cast<uint32_t*>((__nv_bfloat16*)out + (size_t)m * ldo + (rr >> 1)) =
                                    pack_bf16(silu_mul(v.x, v.y), silu_mul(v.z, v.w));
                            } else if (EPI == EPI_PARTIAL) {
                                *reinterpret_cast<float4*>(partial + ((size_t)blockIdx.z * Cc + m) * R + rr) = v;
                            } else if (EPI == EPI_ADD) {
                                float4* dst = reinterpret_cast<float4*>((float*)out + (size_t)m * ldo + rr);
                                float4 a = *dst;
                                a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
                                *dst = a;
                            } else if (sizeof(TO) == 4) {
                                *reinterpret_cast<float4*>((float*)out + (size_t)m * ldo + rr) = v;
                            } else {
                                uint2 pk;
                                pk.x = pack_bf16(v.x, v.y);
                                pk.y = pack_bf16(v.z, v.w);
                                *reinterpret_cast<uint2*>((__nv_bfloat16*)out + (size_t)m * ldo + rr) = pk;
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const int r1 = rr + u;
                                if (r1 >= R) break;
                                if (EPI == EPI_SWIGLU) {
                                    if (!(u & 1)) ((__nv_bfloat16*)out)[(size_t)m * ldo + (r1 >> 1)] = __float2bfloat16_rn(silu_mul(e[u], e[u + 1]));
                                } else if (EPI == EPI_PARTIAL) partial[((size_t)blockIdx.z * Cc + m) * R + r1] = e[u];
                                else if (EPI == EPI_ADD) ((float*)out)[(size_t)m * ldo + r1] += e[u];
                                else if (sizeof(TO) == 4) ((float*)out)[(size_t)m * ldo + r1] = e[u];
                                else ((__nv_bfloat16*)out)[(size_t)m * ldo + r1] = __float2bfloat16_rn(e[u]);
                            }
                        }
                    }
                }
            } else if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += GROUP) {
                if (col0 + c >= Cc) break;                  // uniform: nothing left in this tile
                uint32_t raw[GROUP];
                tmem_ld_group<GROUP>(taddr + c, raw);
                if (EPI == EPI_SWIGLU) {
                    // Rows 2i (gate) and 2i + 1 (up) sit in neighbouring lanes; the even lane finishes the even
                    // tokens of the pair and the odd lane the odd ones, so each lane does half of the work.
                    const int p = lane & 1;
#pragma unroll
                    for (int j = 0; j < GROUP; j += 2) {
                        const float lo = __uint_as_float(raw[j]), hi = __uint_as_float(raw[j + 1]);
                        const float mine = p ? hi : lo;
                        const float theirs = __shfl_xor_sync(0xffffffffu, p ? lo : hi, 1);
                        const int m = col0 + c + j + p;     // token
                        if (m < Cc && r < R)
                            ((__nv_bfloat16*)out)[(size_t)m * ldo + (r >> 1)] =
                                __float2bfloat16_rn(p ? silu_mul(theirs, mine) : silu_mul(mine, theirs));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < GROUP; j++) {
                        const int m = col0 + c + j;         // token
                        const float x = __uint_as_float(raw[j]);
                        if (m < Cc && r < R) {
                            if (EPI == EPI_PARTIAL) partial[((size_t)blockIdx.z * Cc + m) * R + r] = x;
                            else if (EPI == EPI_ADD) ((float*)out)[(size_t)m * ldo + r] += x;
                            else if (sizeof(TO) == 4) ((float*)out)[(size_t)m * ldo + r] = x;
                            else ((__nv_bfloat16*)out)[(size_t)m * ldo + r] = __float2bfloat16_rn(x);
                        }
                    }
                }
            }
            }
            }
        }
    }

    if (*abort_flag) {
        // copies that were issued may still be landing in this block's shared memory
        unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 50000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// ---- persistent kernel for many tokens ---------------------------------------------------------
// One block per SM walks over 128 x 256 output tiles (row tiles fastest, so that the blocks
// running together share a few weight tiles and all of the activations in L2).  Tensor memory
// holds TWO accumulators: while the epilogue warps drain tile i (tensor memory -> a small
// per-warp staging area in shared memory -> coalesced global accesses), the MMA warp already
// fills the other accumulator with tile i+1, fed by the same TMA ring, whose stage and phase
// counters simply run on across tiles.
struct PBarriers {
    unsigned long long full[MAX_STAGES];
    unsigned long long empty[MAX_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int PBN = 256;                 // tile width
constexpr int PCW = 32;                  // columns staged at a time
constexpr int PSP = PCW + 4;             // staging row pitch in floats
constexpr int P_STAGING_BYTES = 4 * 32 * PSP * 4;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Add-into-residual: a chunk's residual values (32 rows x PCW columns, 8 loads of 16 bytes per lane).  The caller asks
// for the NEXT chunk's values before it drains a chunk, so that they travel meanwhile.  (The epilogue of a tile stays
// bound by memory all the same: at a block's last tile all blocks read and write their part of the 32-bit residual
// at once, 128 KB each way per block in 8 to 9 us.)
constexpr int RES_LPR = PCW / 4, RES_RPI = 32 / RES_LPR, RES_N = 32 / RES_RPI;
template <typename TO>
__device__ __forceinline__ void load_residual_chunk(float4 (&res)[RES_N], int c0, int lane, const TO* out, int grow0, int gcol0,
                                                    int rows, int N, int ldo) {
    const int sub = lane / RES_LPR, col = (lane % RES_LPR) * 4;
#pragma unroll
    for (int u = 0; u < RES_N; u++) {
        const int r = RES_RPI * u + sub;
        res[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows && gcol0 + c0 + col < N)
            res[u] = *reinterpret_cast<const float4*>((const float*)out + (size_t)(grow0 + r) * ldo + gcol0 + c0 + col);
    }
}

// drain PCW accumulator columns [c0, c0+PCW) of this warp's 32 rows and apply the epilogue (res: the chunk's residual
// values for add-into-residual, unused otherwise)
template <int EPI, typename TO>
__device__ __forceinline__ void drain_chunk(float* stage, uint32_t taddr, int c0, int lane, TO* out, int grow0, int gcol0,
                                            int rows, int N, int ldo, const float4 (&res)[RES_N]) {
    float* mine = stage + lane * PSP;
    constexpr int ALPR = RES_LPR, ARPI = RES_RPI, ANL = RES_N;
    {
        static_assert(PCW == 32, "one 32-column load from tensor memory per chunk");
        uint32_t raw[32];
        tmem_ld32_raw(taddr + c0, raw);
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(mine + j) = make_float4(__uint_as_float(raw[j]), __uint_as_float(raw[j + 1]),
                                                               __uint_as_float(raw[j + 2]), __uint_as_float(raw[j + 3]));
    }
    __syncwarp();
    const int gc = gcol0 + c0;
    if (EPI == EPI_ADD || (EPI == EPI_STORE && sizeof(TO) == 4)) {
        // PCW/4 lanes x float4 cover a row's columns: ARPI rows per instruction
        const int sub = lane / ALPR, col = (lane % ALPR) * 4;
#pragma unroll
        for (int u = 0; u < ANL; u++) {
            const int r = ARPI * u + sub;
            if (r < rows && gc + col < N) {
                float4 a = *reinterpret_cast<const float4*>(stage + r * PSP + col);
                if (EPI == EPI_ADD) { a.x += res[u].x; a.y += res[u].y; a.z += res[u].z; a.w += res[u].w; }
                *reinterpret_cast<float4*>((float*)out + (size_t)(grow0 + r) * ldo + gc + col) = a;
            }
        }
    } else if (EPI == EPI_SWIGLU) {
        // PCW/8 lanes x 8 accumulator columns (4 gate/up pairs -> 4 outputs) cover a row
        constexpr int LPR = PCW / 8, RPI = 32 / LPR;
        const int sub = lane / LPR, col = (lane % LPR) * 8;
#pragma unroll 2
        for (int rr = 0; rr < rows; rr += RPI) {
            int r = rr + sub;
            if (r < rows && gc + col < N) {
                const float* a = stage + r * PSP + col;
                float4 lo = *reinterpret_cast<const float4*>(a), hi = *reinterpret_cast<const float4*>(a + 4);
                uint2 pk;
                pk.x = pack_bf16(silu_mul(lo.x, lo.y), silu_mul(lo.z, lo.w));
                pk.y = pack_bf16(silu_mul(hi.x, hi.y), silu_mul(hi.z, hi.w));
                *reinterpret_cast<uint2*>((__nv_bfloat16*)out + (size_t)(grow0 + r) * ldo + ((gc + col) >> 1)) = pk;
            }
        }
    } else {
        constexpr int LPR = PCW / 8, RPI = 32 / LPR;
        const int sub = lane / LPR, col = (lane % LPR) * 8;
#pragma unroll 2
        for (int rr = 0; rr < rows; rr += RPI) {
            int r = rr + sub;
            if (r < rows && gc + col < N) {
                const float* a = stage + r * PSP + col;
                float4 lo = *reinterpret_cast<const float4*>(a), hi = *reinterpret_cast<const float4*>(a + 4);
                uint4 pk;
                pk.x = pack_bf16(lo.x, lo.y); pk.y = pack_bf16(lo.z, lo.w);
                pk.z = pack_bf16(hi.x, hi.y); pk.w = pack_bf16(hi.z, hi.w);
                *reinterpret_cast<uint4*>((__nv_bfloat16*)out + (size_t)(grow0 + r) * ldo + gc + col) = pk;
            }
        }
    }
    __syncwarp();                      // the staging rows are rewritten by the next chunk
}

template <int EPI, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                          TO* __restrict__ out, int R, int Cc, int K, int ldo, int stages, int* status) {
    constexpr int Y_TILE_BYTES = PBN * BK * 2;
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 32) { prefetch_map(&map_x); prefetch_map(&map_y); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t xs = base;
    const uint32_t ys = base + (uint32_t)stages * X_TILE_BYTES;
    float* staging = reinterpret_cast<float*>(aligned + (size_t)stages * (X_TILE_BYTES + Y_TILE_BYTES));
    PBarriers* bars = reinterpret_cast<PBarriers*>(aligned + (size_t)stages * (X_TILE_BYTES + Y_TILE_BYTES) + P_STAGING_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_tiles = (R + BM - 1) / BM, col_tiles = (Cc + PBN - 1) / PBN;
    const int n_tiles = row_tiles * col_tiles;
    const int nkb = (K + BK - 1) / BK;
    const int my_tiles = ((int)blockIdx.x < n_tiles) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 4);       // one arrival per epilogue warp
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
    if (!(warp == 0 && lane == 0)) gfb_pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            // Stage, phase and tile coordinates are carried along, not recomputed: this one thread
            // has about 500 cycles per k-block and integer divisions would eat most of them.
            // The ring is primed with weight tiles (no kernel writes weights) before the wait for the
            // previous kernel; the activation tiles of those stages follow it.
            const int total = my_tiles * nkb;
            const int n_pre = total < stages ? total : stages;
            {
                int kb = 0, tile = (int)blockIdx.x;
                for (int it = 0; it < n_pre; it++) {
                    const uint32_t full = smem_u32(&bars->full[it]);
                    mbar_expect_tx(full, X_TILE_BYTES + Y_TILE_BYTES);
                    tma_load_2d(ys + it * Y_TILE_BYTES, &map_y, kb * BK, (tile / row_tiles) * PBN, full);
                    if (++kb == nkb) { kb = 0; tile += (int)gridDim.x; }
                }
            }
            gfb_pdl_wait();
            int kb = 0, tile = (int)blockIdx.x;
            int row0 = (tile % row_tiles) * BM, col0 = (tile / row_tiles) * PBN;
            int s = 0;
            uint32_t ph = 0;
            for (int it = 0; it < total; it++) {
                const uint32_t full = smem_u32(&bars->full[s]);
                if (it < n_pre) {
                    tma_load_2d(xs + s * X_TILE_BYTES, &map_x, kb * BK, row0, full);
                } else {
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag, status, 1)) break;
                    mbar_expect_tx(full, X_TILE_BYTES + Y_TILE_BYTES);
                    tma_load_2d(xs + s * X_TILE_BYTES, &map_x, kb * BK, row0, full);
                    tma_load_2d(ys + s * Y_TILE_BYTES, &map_y, kb * BK, col0, full);
                }
                if (++s == stages) { s = 0; ph ^= 1u; }
                if (++kb == nkb) {
                    kb = 0;
                    tile += (int)gridDim.x;
                    row0 = (tile % row_tiles) * BM;
                    col0 = (tile / row_tiles) * PBN;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BM, PBN);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                const int ab = ti & 1;
                ok = mbar_wait(smem_u32(&bars->acc_empty[ab]), ((uint32_t)(ti >> 1) & 1u) ^ 1u, abort_flag, status, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(ab * PBN);
                for (int kb = 0; kb < nkb; kb++) {
                    ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag, status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = umma_smem_desc(xs + s * X_TILE_BYTES);
                    const uint64_t db = umma_smem_desc(ys + s * Y_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(smem_u32(&bars->empty[s]));
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bars->acc_full[ab]));
            }
        }
    } else {
        const int q = warp & 3;
        float* stage = staging + q * 32 * PSP;
        for (int ti = 0; ti < my_tiles; ti++) {
            const int ab = ti & 1;
            const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
            const int row0 = (tile % row_tiles) * BM, col0 = (tile / row_tiles) * PBN;
            if (!mbar_wait(smem_u32(&bars->acc_full[ab]), (uint32_t)(ti >> 1) & 1u, abort_flag, status, 3)) break;
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * PBN);
            const int rows = min(32, R - (row0 + q * 32));
            float4 res[RES_N], res_next[RES_N];
            if (EPI == EPI_ADD) load_residual_chunk(res, 0, lane, out, row0 + q * 32, col0, rows, Cc, ldo);
#pragma unroll 1
            for (int c0 = 0; c0 < PBN; c0 += PCW) {
                if (col0 + c0 >= Cc) break;
                if (EPI == EPI_ADD) load_residual_chunk(res_next, c0 + PCW, lane, out, row0 + q * 32, col0, c0 + PCW < PBN ? rows : 0, Cc, ldo);
                if (rows > 0) drain_chunk<EPI, TO>(stage, taddr, c0, lane, out, row0 + q * 32, col0, rows, Cc, ldo, res);
                else { float v[16]; for (int c = 0; c < PCW; c += 16) tmem_ld16(taddr + c0 + c, v); }
                if (EPI == EPI_ADD) {
#pragma unroll
                    for (int u = 0; u < RES_N; u++) res[u] = res_next[u];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[ab]));
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

// ---- pairs of SMs: cta_group::2 ---------------------------------------------------------------
// Two blocks of a cluster work as one 256 x 256 tile: each loads its own 128 rows of the
// activations and HALF of the weight tile (128 of the 256 weight rows); one tcgen05.mma issued by
// the leader block multiplies with operands from both blocks' shared memory and writes 128
// accumulator rows into each block's tensor memory.  Per SM this halves the weight-operand traffic
// into and out of shared memory, which is what bounds the one-SM 128 x 256 tile.  No TMA
// multicast is used: every block issues its own loads (with .cta_group::2 so that they may signal
// the leader's barrier).  Barriers: `full` lives in the leader and counts the bytes of both
// blocks' loads; the MMA's commit is multicast to both blocks' `empty` and `acc_full`; both
// blocks' epilogue warps arrive on the leader's `acc_empty`.
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;      // clears the bit that tells the two blocks of a pair apart
constexpr int PAIR_STAGE_BYTES = 2 * X_TILE_BYTES;   // 128 activation rows + 128 weight rows, 64 k each

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {      // arrives on `bar` in both blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int EPI, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                    TO* __restrict__ out, int R, int Cc, int K, int ldo, int stages, int* status) {
    extern __shared__ uint8_t smem_raw[];
    if (threadIdx.x == 32) { prefetch_map(&map_x); prefetch_map(&map_y); }
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t xs = base;
    const uint32_t ys = base + (uint32_t)stages * X_TILE_BYTES;
    float* staging = reinterpret_cast<float*>(aligned + (size_t)stages * PAIR_STAGE_BYTES);
    PBarriers* bars = reinterpret_cast<PBarriers*>(aligned + (size_t)stages * PAIR_STAGE_BYTES + P_STAGING_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    const int row_tiles = (R + 255) / 256, col_tiles = (Cc + 255) / 256;
    const int n_tiles = row_tiles * col_tiles;
    const int nkb = (K + BK - 1) / BK;
    const int my_tiles = pair < n_tiles ? (n_tiles - 1 - pair) / n_pairs + 1 : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 8);       // four epilogue warps in each of the two blocks
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                          // both blocks' barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    gfb_pdl_launch();
    if (!(warp == 0 && lane == 0)) gfb_pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            const int total = my_tiles * nkb;
            // Weights are written by no kernel: the weight halves of the first round of the ring are asked for ahead
            // of the wait for the preceding kernel (fresh barriers: every stage is free), the activations behind it.
            const int n_pre = min(stages, total);
            {
                int kb = 0, tile = pair;
                for (int it = 0; it < n_pre; it++) {
                    const uint32_t full = smem_u32(&bars->full[it]) & PEER_MASK;
                    if (leader) mbar_expect_tx(smem_u32(&bars->full[it]), 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(ys + it * X_TILE_BYTES, &map_y, kb * BK, (tile / row_tiles) * 256 + (int)rank * 128, full);
                    if (++kb == nkb) { kb = 0; tile += n_pairs; }
                }
            }
            gfb_pdl_wait();
            int kb = 0, tile = pair, s = 0;
            uint32_t ph = 0;
            int row0 = (tile % row_tiles) * 256 + (int)rank * 128, wrow0 = (tile / row_tiles) * 256 + (int)rank * 128;
            for (int it = 0; it < total; it++) {
                const uint32_t full = smem_u32(&bars->full[s]) & PEER_MASK;        // the leader's barrier
                if (it >= n_pre) {
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort_flag, status, 1)) break;
                    if (leader) mbar_expect_tx(smem_u32(&bars->full[s]), 2 * PAIR_STAGE_BYTES);
                    tma_load_2d_pair(ys + s * X_TILE_BYTES, &map_y, kb * BK, wrow0, full);
                }
                tma_load_2d_pair(xs + s * X_TILE_BYTES, &map_x, kb * BK, row0, full);
                if (++s == stages) { s = 0; ph ^= 1u; }
                if (++kb == nkb) {
                    kb = 0;
                    tile += n_pairs;
                    row0 = (tile % row_tiles) * 256 + (int)rank * 128;
                    wrow0 = (tile / row_tiles) * 256 + (int)rank * 128;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc(256, 256);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                const int ab = ti & 1;
                ok = mbar_wait(smem_u32(&bars->acc_empty[ab]), ((uint32_t)(ti >> 1) & 1u) ^ 1u, abort_flag, status, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem + (uint32_t)(ab * 256);
                for (int kb = 0; kb < nkb; kb++) {
                    ok = mbar_wait(smem_u32(&bars->full[s]), ph, abort_flag, status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = umma_smem_desc(xs + s * X_TILE_BYTES);
                    const uint64_t db = umma_smem_desc(ys + s * X_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) umma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(smem_u32(&bars->empty[s]));
                    if (++s == stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit_pair(smem_u32(&bars->acc_full[ab]));
            }
        }
    } else {
        const int q = warp & 3;
        float* stage = staging + q * 32 * PSP;
        for (int ti = 0; ti < my_tiles; ti++) {
            const int ab = ti & 1;
            const int tile = pair + ti * n_pairs;
            const int row0 = (tile % row_tiles) * 256 + (int)rank * 128, col0 = (tile / row_tiles) * 256;
            if (!mbar_wait(smem_u32(&bars->acc_full[ab]), (uint32_t)(ti >> 1) & 1u, abort_flag, status, 3)) break;
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(ab * 256);
            const int rows = min(32, R - (row0 + q * 32));
            float4 res[RES_N], res_next[RES_N];
            if (EPI == EPI_ADD) load_residual_chunk(res, 0, lane, out, row0 + q * 32, col0, rows, Cc, ldo);
#pragma unroll 1
            for (int c0 = 0; c0 < 256; c0 += PCW) {
                if (col0 + c0 >= Cc || rows <= 0) break;
                if (EPI == EPI_ADD) load_residual_chunk(res_next, c0 + PCW, lane, out, row0 + q * 32, col0, c0 + PCW < 256 ? rows : 0, Cc, ldo);
                drain_chunk<EPI, TO>(stage, taddr, c0, lane, out, row0 + q * 32, col0, rows, Cc, ldo, res);
                if (EPI == EPI_ADD) {
#pragma unroll
                    for (int u = 0; u < RES_N; u++) res[u] = res_next[u];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&bars->acc_empty[ab]) & PEER_MASK);
        }
    }

    if (*abort_flag) {
        unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 50000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                          // neither block leaves while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// Sum the partials of a split over K in ascending split order and apply the epilogue.
// partial: [S][M][N] f32.
template <int EPI, typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TO* __restrict__ out, int S, int M, int N, int ldo) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    int m = blockIdx.y;
    if (EPI == EPI_SWIGLU) {
        int pair = n;
        if (2 * pair + 1 >= N) return;
        float g = 0.f, u = 0.f;
        for (int s = 0; s < S; s++) {
            const float* p = partial + ((size_t)s * M + m) * N + 2 * pair;
            g += p[0];
            u += p[1];
        }
        ((__nv_bfloat16*)out)[(size_t)m * ldo + pair] = __float2bfloat16_rn(silu_mul(g, u));
    } else {
        if (n >= N) return;
        float acc = 0.f;
        for (int s = 0; s < S; s++) acc += partial[((size_t)s * M + m) * N + n];
        if (EPI == EPI_ADD) ((float*)out)[(size_t)m * ldo + n] += acc;
        else if (sizeof(TO) == 4) ((float*)out)[(size_t)m * ldo + n] = acc;
        else ((__nv_bfloat16*)out)[(size_t)m * ldo + n] = __float2bfloat16_rn(acc);
    }
}

// ---- host side ----------------------------------------------------------------------------
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

// 2-D map over a K-major bf16 matrix [rows, K]: box = 64 k x box_rows rows, 128-byte swizzle,
// zero fill outside (so a ragged K or a ragged last tile contributes zeros).
int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return gfb_fail("gfb_gemm_tc: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gfb_fail("gfb_gemm_tc: cuTensorMapEncodeTiled failed with %d (rows %d, K %d)", (int)r, rows, K);
    return 0;
}

size_t smem_bytes(int bn, int stages) {
    return 1024 + (size_t)stages * (X_TILE_BYTES + bn * BK * 2) + sizeof(Barriers);
}
// the normal orientation stages its 128 x bn accumulator (rows padded by 4 floats) in the ring
size_t staging_bytes(int bn) { return (size_t)BM * (bn + 4) * 4; }

template <int BN, bool SWAP, int EPI, typename TO>
int launch(const CUtensorMap& mx, const CUtensorMap& my, void* out, float* partial, int R, int Cc, int K, int ldo,
           int splits, int kb_per_split, int stages, int* status, cudaStream_t stream) {
    auto kern = gemm_tc_kernel<BN, SWAP, EPI, TO>;
    size_t smem = smem_bytes(BN, stages);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("gfb_gemm_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    dim3 grid((R + BM - 1) / BM, (Cc + BN - 1) / BN, splits);
    cudaError_t e = gfb_launch(kern, grid, dim3(192), smem, stream, mx, my, (TO*)out, partial, R, Cc, K, ldo, kb_per_split, stages, status);
    return gfb_check(e, "gfb_gemm_tc");
}

size_t persistent_smem_bytes(int stages) {
    return 1024 + (size_t)stages * (X_TILE_BYTES + PBN * BK * 2) + P_STAGING_BYTES + sizeof(PBarriers);
}

template <int EPI, typename TO>
int launch_persistent(const CUtensorMap& mx, const CUtensorMap& my, void* out, int R, int Cc, int K, int ldo, int stages,
                      int sm_count, int* status, cudaStream_t stream) {
    auto kern = gemm_tc_persistent_kernel<EPI, TO>;
    size_t smem = persistent_smem_bytes(stages);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("gfb_gemm_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    int tiles = ((R + BM - 1) / BM) * ((Cc + PBN - 1) / PBN);
    dim3 grid(tiles < sm_count ? tiles : sm_count);
    cudaError_t e = gfb_launch(kern, grid, dim3(192), smem, stream, mx, my, (TO*)out, R, Cc, K, ldo, stages, status);
    return gfb_check(e, "gfb_gemm_tc (persistent)");
}

size_t pair_smem_bytes(int stages) {
    return 1024 + (size_t)stages * PAIR_STAGE_BYTES + P_STAGING_BYTES + sizeof(PBarriers);
}

template <int EPI, typename TO>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& my, void* out, int R, int Cc, int K, int ldo, int stages,
                int sm_count, int* status, cudaStream_t stream) {
    auto kern = gemm_tc_pair_kernel<EPI, TO>;
    size_t smem = pair_smem_bytes(stages);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gfb_fail("gfb_gemm_tc: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    int tiles = ((R + 255) / 256) * ((Cc + 255) / 256);
    int pairs = sm_count / 2;
    if (tiles < pairs) pairs = tiles;
    cudaError_t e = gfb_launch_cluster(kern, dim3(2 * pairs), dim3(192), smem, stream, 2u, mx, my, (TO*)out, R, Cc, K, ldo,
                                       stages, status);
    return gfb_check(e, "gfb_gemm_tc (pair)");
}

template <int BN, bool SWAP>
int dispatch_epi(int epi, int out_dt, const CUtensorMap& mx, const CUtensorMap& my, void* out, float* partial, int R,
                 int Cc, int K, int ldo, int splits, int kbps, int stages, int* status, cudaStream_t stream) {
    typedef __nv_bfloat16 bf16;
#define GO(E, T) return launch<BN, SWAP, E, T>(mx, my, out, partial, R, Cc, K, ldo, splits, kbps, stages, status, stream)
    if (epi == EPI_PARTIAL) { if (SWAP) GO(EPI_PARTIAL, float); return gfb_fail("gfb_gemm_tc: a split over K needs the swapped orientation"); }
    if (epi == EPI_ADD) GO(EPI_ADD, float);
    if (epi == EPI_SWIGLU) GO(EPI_SWIGLU, bf16);
    if (epi == EPI_STORE && out_dt == GFB_F32) GO(EPI_STORE, float);
    if (epi == EPI_STORE && out_dt == GFB_BF16) GO(EPI_STORE, bf16);
#undef GO
    return gfb_fail("gfb_gemm_tc: unsupported epilogue %d / output type %d", epi, out_dt);
}

}  // namespace

// out = A[M,K] * W[N,K]^T with the epilogue `epi`.  swap = 0: 128 tokens x bn weight rows per tile
// (bn 128 or 256); swap = 1: 128 weight rows x bn tokens (bn 16, 32, 64 or 128, M <= bn * tiles).
// splits > 1 (swap only) writes partials to `workspace` ([splits, M, N] f32); with reduce != 0 they are
// summed and the epilogue applied by a second kernel, with reduce == 0 the caller's next kernel consumes
// them.  *splits_used receives the number of slices that were written.
GFB_API int gfb_gemm_tc(const void* A, const void* W, void* out, int out_dt, int M, int N, int K, int epi, int swap,
                        int bn, int splits, int stages, float* workspace, int reduce, int* splits_used, int* status,
                        cudaStream_t stream) {
    if (splits_used) *splits_used = 1;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8) return gfb_fail("gfb_gemm_tc: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (N % 8) return gfb_fail("gfb_gemm_tc: N = %d must be a multiple of 8", N);
    if (epi == EPI_SWIGLU && N % 16) return gfb_fail("gfb_gemm_tc: SwiGLU needs N %% 16 == 0, got %d", N);
    if (((uintptr_t)A | (uintptr_t)W | (uintptr_t)out) & 15) return gfb_fail("gfb_gemm_tc: operands must be 16-byte aligned");
    if (stages < 2 || stages > MAX_STAGES) return gfb_fail("gfb_gemm_tc: stages = %d out of range", stages);
    if (bn < 512 && smem_bytes(bn, stages) > 227 * 1024) return gfb_fail("gfb_gemm_tc: %d stages of a %d-column tile exceed shared memory", stages, bn);
    if (!swap && bn < 512 && (size_t)stages * (X_TILE_BYTES + bn * BK * 2) < staging_bytes(bn))
        return gfb_fail("gfb_gemm_tc: %d stages are too few to stage a 128 x %d accumulator", stages, bn);
    const int total_kb = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > total_kb) splits = total_kb;
    int kbps = (total_kb + splits - 1) / splits;
    splits = (total_kb + kbps - 1) / kbps;                 // no empty split
    if (splits_used) *splits_used = splits;
    if (splits > 1 && !swap) return gfb_fail("gfb_gemm_tc: a split over K needs the swapped orientation");
    if (splits > 1 && workspace == nullptr) return gfb_fail("gfb_gemm_tc: a split over K needs a workspace");

    const int ldo = epi == EPI_SWIGLU ? N / 2 : N;
    const int R = swap ? N : M, Cc = swap ? M : N;
    CUtensorMap mx, my;
    if (make_map(&mx, swap ? W : A, R, K, BM)) return 1;
    if (make_map(&my, swap ? A : W, Cc, K, bn >= 512 ? PBN : bn)) return 1;
    const int kernel_epi = splits > 1 ? EPI_PARTIAL : epi;
    int rc;
    if (!swap && bn == 1024) {
        // pairs of SMs: 256 x 256 tiles with cta_group::2
        static int sm_count2 = 0;
        if (sm_count2 == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sm_count2, cudaDevAttrMultiProcessorCount, dev);
        }
        int st = stages;
        while (st > 2 && pair_smem_bytes(st) > 227 * 1024) st--;
        CUtensorMap my2;
        if (make_map(&my2, W, N, K, 128)) return 1;
        typedef __nv_bfloat16 bf16;
        if (epi == EPI_ADD) return launch_pair<EPI_ADD, float>(mx, my2, out, M, N, K, ldo, st, sm_count2, status, stream);
        if (epi == EPI_SWIGLU) return launch_pair<EPI_SWIGLU, bf16>(mx, my2, out, M, N, K, ldo, st, sm_count2, status, stream);
        if (out_dt == GFB_F32) return launch_pair<EPI_STORE, float>(mx, my2, out, M, N, K, ldo, st, sm_count2, status, stream);
        return launch_pair<EPI_STORE, bf16>(mx, my2, out, M, N, K, ldo, st, sm_count2, status, stream);
    }
    if (!swap && bn == 512) {
        // persistent kernel: 128 x 256 tiles, two accumulators in tensor memory
        static int sm_count = 0;
        if (sm_count == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        }
        int st = stages;
        while (st > 2 && persistent_smem_bytes(st) > 227 * 1024) st--;
        CUtensorMap my2;
        if (make_map(&my2, W, N, K, PBN)) return 1;
        typedef __nv_bfloat16 bf16;
        if (epi == EPI_ADD) return launch_persistent<EPI_ADD, float>(mx, my2, out, M, N, K, ldo, st, sm_count, status, stream);
        if (epi == EPI_SWIGLU) return launch_persistent<EPI_SWIGLU, bf16>(mx, my2, out, M, N, K, ldo, st, sm_count, status, stream);
        if (out_dt == GFB_F32) return launch_persistent<EPI_STORE, float>(mx, my2, out, M, N, K, ldo, st, sm_count, status, stream);
        return launch_persistent<EPI_STORE, bf16>(mx, my2, out, M, N, K, ldo, st, sm_count, status, stream);
    }
#define BNCASE(B, S) rc = dispatch_epi<B, S>(kernel_epi, out_dt, mx, my, out, workspace, R, Cc, K, ldo, splits, kbps, stages, status, stream)
    if (!swap && bn == 256) BNCASE(256, false);
    else if (!swap && bn == 128) BNCASE(128, false);
    else if (swap && bn == 16) BNCASE(16, true);
    else if (swap && bn == 32) BNCASE(32, true);
    else if (swap && bn == 64) BNCASE(64, true);
    else if (swap && bn == 128) BNCASE(128, true);
    else return gfb_fail("gfb_gemm_tc: no kernel for swap = %d, bn = %d", swap, bn);
#undef BNCASE
    if (rc) return rc;
    if (splits > 1 && reduce) {
        typedef __nv_bfloat16 bf16;
        int cols = epi == EPI_SWIGLU ? N / 2 : N;
        dim3 grid((cols + 255) / 256, M);
        cudaError_t e;
#define RED(E, T) e = gfb_launch(splitk_reduce_kernel<E, T>, grid, dim3(256), 0, stream, (const float*)workspace, (T*)out, splits, M, N, ldo)
        if (epi == EPI_ADD) RED(EPI_ADD, float);
        else if (epi == EPI_SWIGLU) RED(EPI_SWIGLU, bf16);
        else if (out_dt == GFB_F32) RED(EPI_STORE, float);
        else RED(EPI_STORE, bf16);
#undef RED
        return gfb_check(e, "gfb_gemm_tc (split reduce)");
    }
    return 0;
}

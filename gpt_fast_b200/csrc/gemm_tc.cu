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

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }

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
            const int n_pre = min(stages, nkb);
            for (int i = 0; i < n_pre; i++) {               // fresh barriers: every stage is free
                uint32_t full = smem_u32(&bars->full[i]);
                mbar_expect_tx(full, X_TILE_BYTES + Y_TILE_BYTES);
                if (SWAP) tma_load_2d(xs + i * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full);
                else tma_load_2d(ys + i * Y_TILE_BYTES, &map_y, (kb0 + i) * BK, col0, full);
            }
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
                tma_load_2d(xs + s * X_TILE_BYTES, &map_x, (kb0 + i) * BK, row0, full);
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
        if (ok) {
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
            if constexpr (!SWAP) {
                if (row0 + q * 32 < R)
                    epilogue_rows<BN, EPI == EPI_PARTIAL ? EPI_STORE : EPI, TO>(reinterpret_cast<float*>(aligned), taddr, q, lane,
                                                                                out, row0, col0, R, Cc, ldo);
            } else {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (col0 + c >= Cc) break;                  // uniform: nothing left in this tile
                float v[16];
                tmem_ld16(taddr + c, v);
                {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        int m = col0 + c + j;               // token
                        float x = v[j];
                        if (EPI == EPI_SWIGLU) {
                            float other = __shfl_xor_sync(0xffffffffu, x, 1);
                            if (m < Cc && r < R && !(lane & 1))
                                ((__nv_bfloat16*)out)[(size_t)m * ldo + (r >> 1)] = __float2bfloat16_rn(silu_mul(x, other));
                        } else if (m < Cc && r < R) {
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
    if (smem_bytes(bn, stages) > 227 * 1024) return gfb_fail("gfb_gemm_tc: %d stages of a %d-column tile exceed shared memory", stages, bn);
    if (!swap && (size_t)stages * (X_TILE_BYTES + bn * BK * 2) < staging_bytes(bn))
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
    if (make_map(&my, swap ? A : W, Cc, K, bn)) return 1;
    const int kernel_epi = splits > 1 ? EPI_PARTIAL : epi;
    int rc;
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

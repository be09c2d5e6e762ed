// C[M,N] = A[M,K] * W[N,K]^T on CUDA cores, any M, N, K, both precisions.
//
// This is the product kernel of the true 32-bit path (FFMA only, no tensor
// cores, so no reduced-precision matrix mode) and the fallback of the bfloat16
// path for shapes the tensor-core kernel refuses (rows that are no multiple of
// 16 bytes).  It stands where gpt-fast calls nn.Linear (model.py:195, :215,
// :227, :145).  Each output element is one thread's sum over k = 0..K-1 in
// ascending order, whatever M and the tile position are: a row's result does
// not depend on which other rows are in the batch.
//
// Epilogues: STORE (C = acc, cast), ADD (C is 32-bit, C += acc: the residual
// sum), SWIGLU (W's rows alternate gate, up; C[M, N/2] = silu(gate) * up).
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    gfb_pdl_launch();
    gfb_pdl_wait();
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand, 4 elements per thread; k is the fast index
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int e = threadIdx.x + i * 256;
            int r = e >> 4, k = e & 15;
            int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? gfb_to_f32(A[(size_t)gm * K + gk]) : 0.f;
            Ws[k][r] = (gn < N && gk < K) ? gfb_to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        if (EPI == EPI_SWIGLU) {
            int No = N >> 1;
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                int n = n0 + tx * 4 + j;          // even: gate row, n+1: up row
                if (n + 1 < N) {
                    float g = acc[i][j], u = acc[i][j + 1];
                    float act = g / (1.f + expf(-g));
                    C[(size_t)m * No + (n >> 1)] = gfb_from_f32<TC>(act * u);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int n = n0 + tx * 4 + j;
                if (n >= N) continue;
                size_t o = (size_t)m * N + n;
                if (EPI == EPI_ADD) C[o] = gfb_from_f32<TC>(gfb_to_f32(C[o]) + acc[i][j]);
                else C[o] = gfb_from_f32<TC>(acc[i][j]);
            }
        }
    }
}

template <typename TA, typename TW, typename TC>
static int launch(const void* A, const void* W, void* C, int M, int N, int K, int epi, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return gfb_fail("gfb_gemm_simt: M = %d is too large", M);
    cudaError_t e;
#define GO(E) e = gfb_launch(gemm_simt_kernel<TA, TW, TC, E>, grid, dim3(256), 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N, K)
    if (epi == EPI_STORE) GO(EPI_STORE);
    else if (epi == EPI_ADD) GO(EPI_ADD);
    else if (epi == EPI_SWIGLU) GO(EPI_SWIGLU);
    else return gfb_fail("gfb_gemm_simt: unknown epilogue %d", epi);
#undef GO
    return gfb_check(e, "gfb_gemm_simt");
}

// in_dt: type of A and W; out_dt: type of C (ADD needs 32-bit C).
GFB_API int gfb_gemm_simt(const void* A, const void* W, void* C, int in_dt, int out_dt, int M, int N, int K,
                          int epi, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return gfb_fail("gfb_gemm_simt: K = %d", K);
    if (epi == EPI_ADD && out_dt != GFB_F32) return gfb_fail("gfb_gemm_simt: the residual sum is kept in 32-bit");
    if (epi == EPI_SWIGLU && (N & 1)) return gfb_fail("gfb_gemm_simt: SwiGLU needs an even number of rows, got %d", N);
    typedef __nv_bfloat16 bf16;
    if (in_dt == GFB_F32 && out_dt == GFB_F32) return launch<float, float, float>(A, W, C, M, N, K, epi, stream);
    if (in_dt == GFB_BF16 && out_dt == GFB_BF16) return launch<bf16, bf16, bf16>(A, W, C, M, N, K, epi, stream);
    if (in_dt == GFB_BF16 && out_dt == GFB_F32) return launch<bf16, bf16, float>(A, W, C, M, N, K, epi, stream);
    return gfb_fail("gfb_gemm_simt: unsupported types in %d out %d", in_dt, out_dt);
}

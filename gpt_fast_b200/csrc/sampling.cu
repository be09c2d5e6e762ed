// Next-token choice on the device, one block per row of 32-bit logits.
//
// gpt-fast's sample() (generate.py:40-57): logits / max(temperature, 1e-5);
// with top_k, everything below the k-th largest value becomes -inf (ties with
// it are kept); softmax; then the exponential race argmax(p / q), q ~ Exp(1),
// which draws from p without a host synchronisation.  Here the same steps run
// in one kernel: the k-th largest value comes from a 4-pass radix select over
// the order-preserving integer image of the floats, and q comes from
// Philox4x32-10 keyed by (seed; request id, token index, vocabulary index), so
// a request draws the same tokens alone or in any batch.  The softmax
// denominator is the same for every candidate and is left out of the argmax.
// Greedy choice (temperature 0 in this library) is a plain argmax, lowest
// index on ties.
#include "common.cuh"

#include <cooperative_groups.h>

GFB_DEFINE_LAST_ERROR()

constexpr int THREADS = 512;

__device__ __forceinline__ uint32_t float_key(float x) {       // ascending order of floats
    uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Exp(1) noise for (request, token index, vocabulary index): -log(u), u in (0,1)
__device__ __forceinline__ float race_noise(uint64_t seed, int64_t request, int token_index, int i) {
    uint32_t r[4];
    philox4x32_10((uint32_t)i, (uint32_t)token_index, (uint32_t)(uint64_t)request, (uint32_t)((uint64_t)request >> 32),
                  (uint32_t)seed, (uint32_t)(seed >> 32), r);
    float u = ((float)(r[0] >> 9) + 0.5f) * (1.0f / 8388608.0f);
    return -logf(u);
}

// argmax over (value, index) pairs, larger value wins, lower index on ties
__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__device__ int block_argmax(float v, int i, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        argmax_combine(v, i, ov, oi);
    }
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    if (warp == 0) {
        int nw = blockDim.x >> 5;
        v = lane < nw ? sv[lane] : -INFINITY;
        i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, o);
            int oi = __shfl_xor_sync(0xffffffffu, i, o);
            argmax_combine(v, i, ov, oi);
        }
        if (lane == 0) si[0] = i;
    }
    __syncthreads();
    return si[0];
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * V;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += THREADS) {
        float x = row[i];
        if (x != x) x = -INFINITY;              // NaN never wins
        argmax_combine(v, idx, x, i);
    }
    int best = block_argmax(v, idx, sv, si);
    if (threadIdx.x == 0) out[blockIdx.x] = best == 0x7fffffff ? 0 : best;
}

// temperature / top-k / exponential race.  The token index of row b is
// token_index[index_map[b]] (index_map optional).  noise_out (optional, [B,V]) receives q.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float temp, int top_k,
              uint64_t seed, const uint64_t* __restrict__ seed_dev, const int64_t* __restrict__ request_ids,
              const int* __restrict__ token_index, const int* __restrict__ index_map, float* __restrict__ noise_out) {
    __shared__ unsigned int hist[256];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_remaining;
    gfb_pdl_launch();
    gfb_pdl_wait();
    if (seed_dev != nullptr) seed = *seed_dev;
    const float* row = logits + (size_t)blockIdx.x * V;

    // pivot = k-th largest scaled logit (everything when top_k <= 0 or >= V)
    float pivot = -INFINITY;
    if (top_k > 0 && top_k < V) {
        uint32_t prefix = 0, mask = 0;
        int remaining = top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int i = threadIdx.x; i < 256; i += THREADS) hist[i] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < V; i += THREADS) {
                float x = row[i] / temp;
                if (x != x) x = -INFINITY;                    // NaN never wins, as in the cluster kernel
                uint32_t k = float_key(x);
                if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int left = remaining, bin = 255;
                for (; bin > 0; bin--) {
                    int c = (int)hist[bin];
                    if (c >= left) break;
                    left -= c;
                }
                sh_prefix = prefix | ((uint32_t)bin << shift);
                sh_remaining = left;
            }
            __syncthreads();
            prefix = sh_prefix;
            remaining = sh_remaining;
            mask |= 255u << shift;
            __syncthreads();
        }
        pivot = key_float(prefix);
    }

    // the draw is the Gumbel form of the exponential race, argmax(p_i / q_i) = argmax(x_i - log q_i), exactly as
    // in the cluster kernel below: both kernels give the same token from the same noise, however wide the row
    int64_t request = request_ids ? request_ids[blockIdx.x] : (int64_t)blockIdx.x;
    int tix = token_index ? token_index[index_map ? index_map[blockIdx.x] : blockIdx.x] : 0;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += THREADS) {
        float x = row[i] / temp;
        if (x != x) x = -INFINITY;
        float qn = race_noise(seed, request, tix, i);
        if (noise_out) noise_out[(size_t)blockIdx.x * V + i] = qn;
        if (x >= pivot) argmax_combine(best, best_i, x - logf(qn), i);
    }
    int winner = block_argmax(best, best_i, sv, si);
    if (threadIdx.x == 0) out[blockIdx.x] = winner == 0x7fffffff ? 0 : winner;
}

// ---- the same choices with a cluster of blocks per row ---------------------------------------
// A decode step has few rows and a wide vocabulary: one block per row leaves most of the GPU
// idle.  Here SAMPLE_CLUSTER blocks share a row.  Each thread keeps its logits in registers
// (the row is read from memory once); the radix-select histograms and the final candidates are
// exchanged through distributed shared memory.  The draw itself is the Gumbel form of the
// exponential race: argmax(p_i / q_i) = argmax(x_i - log q_i), so neither the maximum nor the
// softmax sum is needed.  Rows wider than SAMPLE_CLUSTER * THREADS * SAMPLE_REGS use the
// one-block kernels above.
constexpr int SAMPLE_CLUSTER = 8;
constexpr int SAMPLE_REGS = 32;

template <bool GREEDY>
__global__ void __launch_bounds__(THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float temp, int top_k,
                      uint64_t seed, const uint64_t* __restrict__ seed_dev, const int64_t* __restrict__ request_ids,
                      const int* __restrict__ token_index, const int* __restrict__ index_map,
                      float* __restrict__ noise_out) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ unsigned int hist[2][256];                     // two histograms in turn: one cluster barrier per pass
    __shared__ unsigned int total[256];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float cand_v;
    __shared__ int cand_i;
    __shared__ float win_v;
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_remaining;
    gfb_pdl_launch();
    gfb_pdl_wait();
    if (seed_dev != nullptr) seed = *seed_dev;
    const int rowi = blockIdx.y;
    const int rank = (int)cluster.block_rank();
    const int lane = threadIdx.x & 31;
    const float* row = logits + (size_t)rowi * V;
    // element e of this thread: index (e * SAMPLE_CLUSTER + rank) * THREADS + tid  (coalesced per block)
    float x[SAMPLE_REGS];
#pragma unroll
    for (int e = 0; e < SAMPLE_REGS; e++) {
        int i = (e * SAMPLE_CLUSTER + rank) * THREADS + threadIdx.x;
        float v = i < V ? row[i] : -INFINITY;
        if (v != v) v = -INFINITY;
        x[e] = GREEDY ? v : v / temp;
    }
    float pivot = -INFINITY;
    if (!GREEDY && top_k > 0 && top_k < V) {
        uint32_t prefix = 0, mask = 0;
        int remaining = top_k;
        for (int i = threadIdx.x; i < 256; i += THREADS) hist[0][i] = 0;
        __syncthreads();
        int pass = 0;
        for (int shift = 24; shift >= 0; shift -= 8, pass++) {
            unsigned int* h = hist[pass & 1];
#pragma unroll
            for (int e = 0; e < SAMPLE_REGS; e++) {
                int i = (e * SAMPLE_CLUSTER + rank) * THREADS + threadIdx.x;
                const uint32_t k = float_key(x[e]);
                const bool in = i < V && (k & mask) == prefix;
                const uint32_t bin = (k >> shift) & 255u;
                if (in) atomicAdd(&h[bin], 1u);
            }
            cluster.sync();                                   // every block's histogram is complete
            // the other histogram, for the next pass: the cluster's blocks read it before they came to this barrier
            for (int i = threadIdx.x; i < 256; i += THREADS) hist[(pass & 1) ^ 1][i] = 0;
            if (threadIdx.x < 256) {
                unsigned int sum = 0;
#pragma unroll
                for (int r = 0; r < SAMPLE_CLUSTER; r++) sum += cluster.map_shared_rank(h, r)[threadIdx.x];
                total[threadIdx.x] = sum;
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                // the highest bin b with count(bins >= b) >= remaining: lane l holds bins [8 l, 8 l + 8)
                unsigned int c[8], mine = 0;
#pragma unroll
                for (int i = 0; i < 8; i++) { c[i] = total[lane * 8 + i]; mine += c[i]; }
                unsigned int above = mine;                    // inclusive sum over this and the higher lanes
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    unsigned int t = __shfl_down_sync(0xffffffffu, above, o);
                    if (lane + o < 32) above += t;
                }
                const bool here = above >= (unsigned int)remaining && above - mine < (unsigned int)remaining;
                const unsigned int who = __ballot_sync(0xffffffffu, here);
                if (who == 0) {                               // fewer elements than remaining (cannot happen with top_k < V)
                    if (lane == 0) { sh_prefix = prefix; sh_remaining = remaining; }
                } else if (here) {
                    int left = remaining - (int)(above - mine), bin = 7;
                    for (; bin > 0; bin--) {
                        if ((int)c[bin] >= left) break;
                        left -= (int)c[bin];
                    }
                    sh_prefix = prefix | ((uint32_t)(lane * 8 + bin) << shift);
                    sh_remaining = left;
                }
            }
            __syncthreads();
            prefix = sh_prefix;
            remaining = sh_remaining;
            mask |= 255u << shift;
        }
        pivot = key_float(prefix);
    }
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    if (GREEDY) {
#pragma unroll
        for (int e = 0; e < SAMPLE_REGS; e++) {
            int i = (e * SAMPLE_CLUSTER + rank) * THREADS + threadIdx.x;
            if (i < V) argmax_combine(best, best_i, x[e], i);
        }
    } else {
        const int64_t request = request_ids ? request_ids[rowi] : (int64_t)rowi;
        const int tix = token_index ? token_index[index_map ? index_map[rowi] : rowi] : 0;
#pragma unroll
        for (int e = 0; e < SAMPLE_REGS; e++) {
            int i = (e * SAMPLE_CLUSTER + rank) * THREADS + threadIdx.x;
            if (i < V && (x[e] >= pivot || noise_out != nullptr)) {      // noise only where it can matter: the survivors
                float qn = race_noise(seed, request, tix, i);
                if (noise_out) noise_out[(size_t)rowi * V + i] = qn;
                if (x[e] >= pivot) argmax_combine(best, best_i, x[e] - logf(qn), i);
            }
        }
    }
    int wi = block_argmax(best, best_i, sv, si);
    if (best_i == wi && wi != 0x7fffffff) win_v = best;       // the thread that holds the block's winner
    __syncthreads();
    if (threadIdx.x == 0) { cand_i = wi; cand_v = (wi == 0x7fffffff) ? -INFINITY : win_v; }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int r = 0; r < SAMPLE_CLUSTER; r++)
            argmax_combine(bv, bi, *cluster.map_shared_rank(&cand_v, r), *cluster.map_shared_rank(&cand_i, r));
        out[rowi] = bi == 0x7fffffff ? 0 : bi;
    }
    cluster.sync();
}

GFB_API int gfb_argmax(const float* logits, int* out, int B, int V, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return gfb_fail("gfb_argmax: V = %d", V);
    cudaError_t e;
    if (V <= SAMPLE_CLUSTER * THREADS * SAMPLE_REGS && B <= 65535)
        e = gfb_launch_cluster(sample_cluster_kernel<true>, dim3(SAMPLE_CLUSTER, B), dim3(THREADS), 0, stream, SAMPLE_CLUSTER,
                               logits, out, V, 1.0f, 0, (uint64_t)0, (const uint64_t*)nullptr, (const int64_t*)nullptr,
                               (const int*)nullptr, (const int*)nullptr, (float*)nullptr);
    else
        e = gfb_launch(argmax_kernel, dim3(B), dim3(THREADS), 0, stream, logits, out, V);
    return gfb_check(e, "gfb_argmax");
}

// seed_dev (optional): the seed is read from device memory instead (so that a captured graph can be
// replayed with another seed).
GFB_API int gfb_sample(const float* logits, int* out, int B, int V, float temperature, int top_k,
                       unsigned long long seed, const unsigned long long* seed_dev, const long long* request_ids,
                       const int* token_index, const int* index_map, float* noise_out, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (V <= 0) return gfb_fail("gfb_sample: V = %d", V);
    float t = temperature > 1e-5f ? temperature : 1e-5f;
    cudaError_t e;
    if (V <= SAMPLE_CLUSTER * THREADS * SAMPLE_REGS && B <= 65535)
        e = gfb_launch_cluster(sample_cluster_kernel<false>, dim3(SAMPLE_CLUSTER, B), dim3(THREADS), 0, stream, SAMPLE_CLUSTER,
                               logits, out, V, t, top_k, (uint64_t)seed, (const uint64_t*)seed_dev, (const int64_t*)request_ids,
                               token_index, index_map, noise_out);
    else
        e = gfb_launch(sample_kernel, dim3(B), dim3(THREADS), 0, stream, logits, out, V, t, top_k, (uint64_t)seed,
                       (const uint64_t*)seed_dev, (const int64_t*)request_ids, token_index, index_map, noise_out);
    return gfb_check(e, "gfb_sample");
}

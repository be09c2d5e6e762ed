// Next-token choice on the device, one block per row of 32-bit logits.
//
// gpt-fast's sample() (generate.py:40-57): logits / max(temperature, 1e-5);
// with top_k, everything below the k-th largest value becomes -inf (ties with
// it are kept); softmax; then the exponential race argmax(p / q), q ~ Exp(1),
// which draws from p without a host synchronisation.  Here the same steps run
// in one kernel: the k-th largest value is found among the few entries above a
// threshold taken from the row's mean and deviation (or by a radix select over
// the order-preserving integer image of the floats), and q comes from
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

// ---- temperature / top-k / exponential race, one block per row ------------------------------------
// The token index of row b is token_index[index_map[b]] (index_map optional).  noise_out (optional, [B,V])
// receives q for every entry.
//
// With top_k far below V (200 of 128,256) nearly all of a row is dropped, so the row is not sorted or
// histogrammed: a first pass over it takes the mean and the deviation of the scaled logits, a second pass
// gathers the entries above mean + z * deviation into shared memory, z chosen so that a normal distribution
// would leave about twice top_k of them.  If that leaves at least top_k and no more than ROW_CAP entries
// (else the threshold is moved and the pass repeated, a few times), the k-th largest value, the survivors and
// the race are settled among those few hundred entries in shared memory (a bitonic sort of their values gives the k-th).  The result does not depend on the
// threshold: it only decides which entries are looked at more closely.  A row that defeats this (fewer
// finite entries than top_k, thousands of equal values around the k-th, a deviation that is not finite) takes
// the slow road: a 4-pass radix select over the whole row in global memory.
constexpr int ROW_THREADS = 1024;
constexpr int ROW_CAP = 2048;
constexpr int ROW_TRIES = 6;
constexpr int ROW_SAMPLE = 16384;

// z with P(N(0,1) > z) = p for 0 < p <= 0.5 (Abramowitz & Stegun 26.2.23, absolute error below 4.5e-4)
__device__ __forceinline__ float normal_tail_z(float p) {
    const float t = sqrtf(-2.f * logf(p));
    return t - (2.515517f + t * (0.802853f + t * 0.010328f)) / (1.f + t * (1.432788f + t * (0.189269f + t * 0.001308f)));
}

// f(index, raw logit) for entries [0, upto) of the row.  Where the row allows 16-byte loads
// a thread has four of them in flight at a time: one block reads the whole row, and it is the latency of the
// loads, not their number, that decides how long that takes.
template <typename F>
__device__ __forceinline__ void for_row(const float* __restrict__ row, int upto, F f) {
    if ((upto & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        constexpr int U = 4;
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = upto >> 2;
        for (int base = 0; base < n4; base += ROW_THREADS * U) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = base + u * ROW_THREADS + threadIdx.x;
                if (i < n4) v[u] = __ldg(r4 + i);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = base + u * ROW_THREADS + threadIdx.x;
                if (i < n4) {
                    const float a[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int j = 0; j < 4; j++) f(4 * i + j, a[j]);
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < upto; i += ROW_THREADS) f(i, row[i]);
    }
}

// what the race works on: the logit over the temperature, an entry that is not a number read as -inf
__device__ __forceinline__ float scaled_logit(float raw, float temp) { return raw != raw ? -INFINITY : raw / temp; }

// the k-th largest scaled logit of the row by a radix select over global memory (8 bits per pass)
__device__ float row_radix_pivot(const float* __restrict__ row, int V, float temp, int top_k, unsigned int* hist,
                                 uint32_t* sh_prefix, int* sh_remaining) {
    uint32_t prefix = 0, mask = 0;
    int remaining = top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += ROW_THREADS) hist[i] = 0;
        __syncthreads();
        for_row(row, V, [&](int, float raw) {
            const uint32_t k = float_key(scaled_logit(raw, temp));
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
        });
        __syncthreads();
        if (threadIdx.x == 0) {
            int left = remaining, bin = 255;
            for (; bin > 0; bin--) {
                int c = (int)hist[bin];
                if (c >= left) break;
                left -= c;
            }
            *sh_prefix = prefix | ((uint32_t)bin << shift);
            *sh_remaining = left;
        }
        __syncthreads();
        prefix = *sh_prefix;
        remaining = *sh_remaining;
        mask |= 255u << shift;
        __syncthreads();
    }
    return key_float(prefix);
}

__global__ void __launch_bounds__(ROW_THREADS)
sample_row_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, float temp, int top_k,
                  uint64_t seed, const uint64_t* __restrict__ seed_dev, const int64_t* __restrict__ request_ids,
                  const int* __restrict__ token_index, const int* __restrict__ index_map, float* __restrict__ noise_out) {
    __shared__ float cand_v[ROW_CAP];
    __shared__ float sort_v[ROW_CAP];
    __shared__ int cand_i[ROW_CAP];
    __shared__ unsigned int hist[256];
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_remaining;
    __shared__ int n_cand;
    __shared__ float sh_pivot;
    gfb_pdl_launch();
    gfb_pdl_wait();
    if (seed_dev != nullptr) seed = *seed_dev;
    const float* row = logits + (size_t)blockIdx.x * V;
    const int64_t request = request_ids ? request_ids[blockIdx.x] : (int64_t)blockIdx.x;
    const int tix = token_index ? token_index[index_map ? index_map[blockIdx.x] : blockIdx.x] : 0;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const bool filter = top_k > 0 && top_k < V;
    bool gathered = false;                                   // uniform: the survivors are among cand_*[0 .. n)
    int n = 0;
    if (filter && top_k <= ROW_CAP / 2) {
        // mean and deviation of the finite entries of a sample of the row: ROW_SAMPLE entries spread evenly over it
        // (in groups of four; tokenizers put frequent tokens at low ids, so a prefix of the row could be far from
        // typical).  A poor guess only costs a repeated pass.
        float s1 = 0.f, s2 = 0.f, cnt = 0.f;
        const int groups = V >> 2;                                   // whole groups of four entries
        const int n_groups = groups < ROW_SAMPLE / 4 ? groups : ROW_SAMPLE / 4;
        const int n_sample = n_groups > 0 ? 4 * n_groups : V;
        if (n_groups > 0) {
            const int stride = groups / n_groups;                    // >= 1
            const bool aligned16 = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
            float x4[ROW_SAMPLE / 4 / ROW_THREADS][4];
#pragma unroll
            for (int j = 0; j < ROW_SAMPLE / 4 / ROW_THREADS; j++) {
                const int gi = threadIdx.x + j * ROW_THREADS;
                if (gi >= n_groups) {
#pragma unroll
                    for (int e = 0; e < 4; e++) x4[j][e] = INFINITY;
                } else if (aligned16) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(row) + (size_t)gi * stride);
                    x4[j][0] = v.x; x4[j][1] = v.y; x4[j][2] = v.z; x4[j][3] = v.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; e++) x4[j][e] = row[(size_t)gi * stride * 4 + e];
                }
            }
#pragma unroll
            for (int j = 0; j < ROW_SAMPLE / 4 / ROW_THREADS; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float x = x4[j][e];
                    if (fabsf(x) < INFINITY) { s1 += x; s2 += x * x; cnt += 1.f; }
                }
        } else {
            for (int i = threadIdx.x; i < V; i += ROW_THREADS) {
                const float x = row[i];
                if (fabsf(x) < INFINITY) { s1 += x; s2 += x * x; cnt += 1.f; }
            }
        }
        s1 = gfb_block_sum(s1, sv);
        s2 = gfb_block_sum(s2, sv);
        cnt = gfb_block_sum(cnt, sv);
        const float mean = s1 / fmaxf(cnt, 1.f);
        const float dev = sqrtf(fmaxf(s2 / fmaxf(cnt, 1.f) - mean * mean, 0.f));
        const float finite = cnt * ((float)V / (float)n_sample);          // estimate for the whole row
        if (cnt >= 2.f && finite >= (float)top_k && dev < INFINITY) {
            float z = normal_tail_z(fminf(0.25f, 2.f * (float)top_k / finite));
            float z_few = INFINITY, z_many = -INFINITY;     // thresholds known to leave too few / too many
            for (int attempt = 0; attempt < ROW_TRIES && !gathered; attempt++) {
                const float tau = mean + z * dev;           // on the raw logits (the temperature is positive)
                __syncthreads();
                if (threadIdx.x == 0) n_cand = 0;
                __syncthreads();
                for_row(row, V, [&](int i, float x) {
                    if (x >= tau) {                             // false for an entry that is not a number
                        const int slot = atomicAdd(&n_cand, 1);
                        if (slot < ROW_CAP) { cand_v[slot] = x / temp; cand_i[slot] = i; }
                    }
                });
                __syncthreads();
                n = n_cand;
                if (n >= top_k && n <= ROW_CAP) gathered = true;
                else if (n < top_k) { z_few = z; z = z_many > -INFINITY ? 0.5f * (z + z_many) : z - 1.f; }
                else { z_many = z; z = z_few < INFINITY ? 0.5f * (z + z_few) : z + 0.5f; }
            }
        }
    }
    if (gathered) {
        // the k-th largest among the gathered entries: a bitonic sort (descending) of a copy of their values,
        // padded with -inf to a power of two
        int N = 32;
        while (N < n) N <<= 1;
        for (int j = threadIdx.x; j < N; j += ROW_THREADS) sort_v[j] = j < n ? cand_v[j] : -INFINITY;
        __syncthreads();
        for (int k2 = 2; k2 <= N; k2 <<= 1) {
            for (int j = k2 >> 1; j > 0; j >>= 1) {
                for (int i = threadIdx.x; i < N; i += ROW_THREADS) {
                    const int l = i ^ j;
                    if (l > i) {
                        const float a = sort_v[i], c = sort_v[l];
                        const bool descending = (i & k2) == 0;
                        if (descending ? a < c : a > c) { sort_v[i] = c; sort_v[l] = a; }
                    }
                }
                __syncthreads();
            }
        }
        if (threadIdx.x == 0) sh_pivot = sort_v[top_k - 1];
        __syncthreads();
        const float pivot = sh_pivot;
        for (int j = threadIdx.x; j < n; j += ROW_THREADS) {
            const float v = cand_v[j];
            if (v >= pivot) argmax_combine(best, best_i, v - logf(race_noise(seed, request, tix, cand_i[j])), cand_i[j]);
        }
        if (noise_out != nullptr)
            for (int i = threadIdx.x; i < V; i += ROW_THREADS) noise_out[(size_t)blockIdx.x * V + i] = race_noise(seed, request, tix, i);
    } else {
        // the draw is the Gumbel form of the exponential race, argmax(p_i / q_i) = argmax(x_i - log q_i), exactly as
        // in the cluster kernel below: all kernels give the same token from the same noise
        float pivot = -INFINITY;
        if (filter) pivot = row_radix_pivot(row, V, temp, top_k, hist, &sh_prefix, &sh_remaining);
        for_row(row, V, [&](int i, float raw) {
            const float x = scaled_logit(raw, temp);
            if (x >= pivot || noise_out != nullptr) {
                const float qn = race_noise(seed, request, tix, i);
                if (noise_out) noise_out[(size_t)blockIdx.x * V + i] = qn;
                if (x >= pivot) argmax_combine(best, best_i, x - logf(qn), i);
            }
        });
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
    // top_k far below V: one block per row gathers the few entries that matter (any number of rows at once);
    // otherwise a cluster of blocks per row where the row fits its registers, else one block per row
    const bool few = top_k > 0 && top_k < V && top_k <= ROW_CAP / 2;
    if (!few && V <= SAMPLE_CLUSTER * THREADS * SAMPLE_REGS && B <= 65535)
        e = gfb_launch_cluster(sample_cluster_kernel<false>, dim3(SAMPLE_CLUSTER, B), dim3(THREADS), 0, stream, SAMPLE_CLUSTER,
                               logits, out, V, t, top_k, (uint64_t)seed, (const uint64_t*)seed_dev, (const int64_t*)request_ids,
                               token_index, index_map, noise_out);
    else
        e = gfb_launch(sample_row_kernel, dim3(B), dim3(ROW_THREADS), 0, stream, logits, out, V, t, top_k, (uint64_t)seed,
                       (const uint64_t*)seed_dev, (const int64_t*)request_ids, token_index, index_map, noise_out);
    return gfb_check(e, "gfb_sample");
}

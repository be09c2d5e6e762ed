// Shared declarations of the sm_100a kernel libraries.
//
// Every library exports plain C functions (called from Python through ctypes):
// raw device pointers, sizes, a stream; the return value is 0 on success and
// `gfb_last_error()` of the same library then explains a failure.  Kernels
// never trap: a condition found on the device (token id out of range, a
// position beyond the cache, a wait that ran out) is written to the caller's
// `status` words and the offending access is skipped.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define GFB_API extern "C" __attribute__((visibility("default")))

// element types of tensors that come in two precisions
enum { GFB_F32 = 0, GFB_BF16 = 1 };

// device status codes: status[0] = first code seen, status[1..3] = details
enum {
    GFB_OK = 0,
    GFB_ERR_TOKEN_RANGE = 1,      // status[1] = token index, status[2] = id
    GFB_ERR_CACHE_RANGE = 2,      // status[1] = token index, status[2] = position
    GFB_ERR_WAIT_TIMEOUT = 3,     // status[1] = which wait, status[2] = block
    GFB_ERR_PAGE_TABLE = 4,       // status[1] = slot, status[2] = page index
};

__device__ __forceinline__ void gfb_report(int* status, int code, int a, int b) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = a;
        status[2] = b;
    }
}

// ---- host side error text ----------------------------------------------------
static thread_local char gfb_error_text[512] = "";

static inline int gfb_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(gfb_error_text, sizeof(gfb_error_text), fmt, ap);
    va_end(ap);
    return 1;
}

static inline int gfb_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gfb_fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

#define GFB_DEFINE_LAST_ERROR() \
    GFB_API const char* gfb_last_error() { return gfb_error_text; }

// ---- launches with programmatic dependent launch -----------------------------------
// Every kernel of the library is launched with the attribute that lets it start
// while its predecessor in the stream is still draining: its blocks become
// resident, set up (barriers, tensor memory, prefetch of weights, which no
// earlier kernel writes) and then wait in `gfb_pdl_wait()` until the
// predecessor has completed and its writes are visible.  A kernel calls
// `gfb_pdl_launch()` once it holds the resources it needs, which allows its own
// successor to become resident.  Because every block of every kernel executes
// the wait before it touches anything an earlier kernel wrote, completion stays
// ordered along the whole chain.  GFB_NO_PDL=1 in the environment turns the
// attribute off (the two instructions are then no-ops).
__device__ __forceinline__ void gfb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void gfb_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool gfb_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("GFB_NO_PDL");
        on = (e != nullptr && e[0] == '1') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t gfb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gfb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with a thread-block cluster of `cluster_x` blocks along x (grid.x must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t gfb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                             unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = gfb_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int gfb_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) return gfb_fail("%s: %s", what, cudaGetErrorString(e));
    return gfb_check_launch(what);
}

// ---- conversions ---------------------------------------------------------------
template <typename T> __device__ __forceinline__ float gfb_to_f32(T v);
template <> __device__ __forceinline__ float gfb_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float gfb_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T gfb_from_f32(float v);
template <> __device__ __forceinline__ float gfb_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 gfb_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- deterministic block reductions (fixed tree, result in every thread) ---------
__device__ __forceinline__ float gfb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float gfb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// `scratch` needs 32 floats of shared memory; blockDim.x must be a multiple of 32.
__device__ __forceinline__ float gfb_block_sum(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = gfb_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? scratch[lane] : 0.f;
    return gfb_warp_sum(r);
}
__device__ __forceinline__ float gfb_block_max(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = gfb_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? scratch[lane] : -INFINITY;
    return gfb_warp_max(r);
}

// ---- the batch of one step, as kernels see it --------------------------------------
// n sequences, T packed tokens.  Token t belongs to sequence tok_seq[t]; the
// sequence's tokens are cu_seqlens[s] .. cu_seqlens[s+1]-1; its cache slot is
// slots[s]; lengths[slot] tokens were cached BEFORE this step, so token t sits
// at position lengths[slot] + (t - cu_seqlens[s]).
struct GfbBatch {
    const int* cu_seqlens;   // [n+1]
    const int* tok_seq;      // [T]
    const int* slots;        // [n]
    const int* lengths;      // [n_slots]
    int n_seqs;
    int n_tokens;
};

// Paged key/value storage of one cache entry: page p of a pool holds
// [n_kv][page_size][head_dim]; page_table[slot][i] is the page that holds the
// slot's positions i*page_size .. (i+1)*page_size-1.
struct GfbPagedKV {
    void* k_pool;
    void* v_pool;
    const int* page_table;   // [n_slots][max_pages]
    int max_pages;
    int page_size;
    int n_pages;
};

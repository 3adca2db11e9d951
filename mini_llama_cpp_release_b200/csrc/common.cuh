// Shared helpers of the sm_100a kernels: element types, loads and stores that widen to
// float, warp and block reductions, and the C entry points' return convention.
//
// Every entry point is `extern "C" int mlc_<name>(..., void* stream)`: it validates its
// sizes on the host, launches on the given stream and returns 0, or returns a negative
// MLC_ERR_* code for a refused size or a positive cudaError_t for a failed launch.  The
// Python side turns non-zero into an exception; nothing falls back to another path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MLC_ERR_BAD_DTYPE (-1)
#define MLC_ERR_BAD_SIZE (-2)
#define MLC_ERR_UNSUPPORTED (-3)

#define MLC_DTYPE_F32 0
#define MLC_DTYPE_BF16 1

#define MLC_LAUNCH_CHECK()                              \
    do {                                                \
        cudaError_t e_ = cudaGetLastError();            \
        if (e_ != cudaSuccess) return (int)e_;          \
    } while (0)

// Per-phase time stamps inside the large kernels are a tuning aid: they are compiled in only with -DMLC_PHASE_STAMPS,
// which the package's own build does not set; without it the pointers that would receive them are ignored.
#ifdef MLC_PHASE_STAMPS
#define MLC_STAMPS_OR_NULL(expr) (expr)
#else
#define MLC_STAMPS_OR_NULL(expr) nullptr
#endif

namespace mlc {

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched through launch_pdl may start while the kernel before it on the stream is still
// running; it must call grid_dependency_wait() before it reads anything an earlier kernel wrote
// (the wait returns once every earlier kernel has finished and its writes are visible), and it
// calls grid_launch_dependents() to let the kernel after it start in the same way.  The launch
// latency of a chain of short kernels then overlaps with their execution.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whether kernels are launched with the programmatic-serialization attribute (one switch per library).
inline int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats of shared memory.
// Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int n_warps = (blockDim.x + 31) >> 5;
    float t = (lane < n_warps) ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int n_warps = (blockDim.x + 31) >> 5;
    float t = (lane < n_warps) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// Where the keys and values of one cache entry live: pools of pages of `page_size`
// tokens, [entry][page][kv_head][token in page][head_dim], and each sequence's list of
// pages.  A negative page number marks a page that was never given or was given back.
struct PagedKV {
    void* k_pool;
    void* v_pool;
    const int* page_table;      // [n_seqs][pages_per_seq]
    long long entry_offset;     // elements from the pool's start to this entry's first page
    int pages_per_seq;
    int page_size;
    int kv_heads;
    int head_dim;
};

__device__ __forceinline__ long long paged_offset(const PagedKV& c, int seq, int pos, int kv_head) {
    const int page = c.page_table[(long long)seq * c.pages_per_seq + pos / c.page_size];
    return c.entry_offset +
           (((long long)page * c.kv_heads + kv_head) * c.page_size + (pos % c.page_size)) * c.head_dim;
}

}  // namespace mlc

// The allocation-free variant of the split-key attention; see attention_noalloc.h for who
// it is for, what it costs and what a caller must keep in mind.
//
// It launches the very kernels of attention_simt.cu (included below for their definitions
// only) and differs in one thing: the partial results go to the array `noalloc_scratch`
// of this file instead of caller-provided memory.
#define MLC_KERNELS_ONLY
#include "attention_simt.cu"
#include "attention_noalloc.h"

#include <mutex>

// Scratch for the partial results of all calls: [rows * n_splits][2] maxima and sums first,
// then [rows * n_splits][head_dim] weighted values.  Device code could name this array
// directly; host code below must not pass the name itself to a kernel (in host code it is a
// stand-in, not a device address) and asks the runtime for the address instead.
static __device__ __align__(256) float noalloc_scratch[MLC_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
std::mutex setup_lock;
float* scratch_on_device[MAX_DEVICES] = {};      // device address of noalloc_scratch, per device, once known

// The array's address on the current device, looked up at the first call on that device.
int scratch_address(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return MLC_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(setup_lock);
    if (scratch_on_device[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, noalloc_scratch);     // with `dev` current: its copy of the array
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return MLC_ERR_UNSUPPORTED;
        scratch_on_device[dev] = p;
    }
    *ptr = scratch_on_device[dev];
    return 0;
}

}  // namespace

extern "C" int mlc_attention_split_noalloc(const void* q, void* out, int dtype, const int* cu_seqlens,
                                           const int* start_pos, int n_seqs, int n_tokens, int max_q_len, int q_heads,
                                           int kv_heads, int hd, float scale, int window, int n_splits, void* k_pool,
                                           void* v_pool, const int* page_table, long long entry_offset,
                                           int pages_per_seq, int page_size, void* stream) {
    using namespace mlc;
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (hd <= 0 || hd > ATT_MAX_HD || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return MLC_ERR_BAD_SIZE;
    if (n_splits < 1 || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    if (dtype != MLC_DTYPE_F32 && dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    const long long rows = (long long)n_tokens * q_heads * n_splits;
    if (rows * (hd + 2) > (long long)MLC_NOALLOC_SCRATCH_FLOATS) return MLC_ERR_BAD_SIZE;   // beyond the fixed array: refuse

    float* scratch = nullptr;
    const int rc = scratch_address(&scratch);
    if (rc != 0) return rc;
    float* part_ml = scratch;                 // rows * 2 floats
    float* part_o = scratch + rows * 2;       // rows * hd floats

    AttnArgs a;
    a.q = q;
    a.out = out;
    a.cu_seqlens = cu_seqlens;
    a.start_pos = start_pos;
    a.part_ml = part_ml;
    a.part_o = part_o;
    a.scale = scale;
    a.q_heads = q_heads;
    a.group = q_heads / kv_heads;
    a.window = window;
    a.heads_per_block = a.group < ATT_ROWS ? a.group : ATT_ROWS;
    a.tokens_per_block = ATT_ROWS / a.heads_per_block;
    a.head_chunks = (a.group + a.heads_per_block - 1) / a.heads_per_block;
    a.n_splits = n_splits;
    const long long gy = (long long)kv_heads * a.head_chunks * n_splits;
    if (gy > 65535) return MLC_ERR_BAD_SIZE;
    PagedKV c{k_pool, v_pool, page_table, entry_offset, pages_per_seq, page_size, kv_heads, hd};
    dim3 grid((max_q_len + a.tokens_per_block - 1) / a.tokens_per_block, (unsigned)gy, n_seqs);
    const size_t smem = (size_t)(ATT_ROWS * hd + ATT_TILE * (hd + 1) + ATT_TILE * hd) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (smem > 48 * 1024) {
        cudaError_t e = (dtype == MLC_DTYPE_F32)
            ? cudaFuncSetAttribute(attention_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
            : cudaFuncSetAttribute(attention_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // With one split the first kernel writes `out` itself and no scratch is touched; with more,
    // every (row, split) pair of the scratch is written here before the merge below reads it.
    if (dtype == MLC_DTYPE_F32)
        attention_simt_kernel<float><<<grid, ATT_WARPS * 32, smem, s>>>(a, c);
    else
        attention_simt_kernel<bf16><<<grid, ATT_WARPS * 32, smem, s>>>(a, c);
    MLC_LAUNCH_CHECK();
    if (n_splits > 1) {
        const long long n_rows = (long long)n_tokens * q_heads;
        const unsigned blocks = (unsigned)((n_rows + 3) / 4);
        if (dtype == MLC_DTYPE_F32)
            attention_combine_kernel<float><<<blocks, 128, 0, s>>>(part_ml, part_o, n_rows, n_splits, hd, (float*)out);
        else
            attention_combine_kernel<bf16><<<blocks, 128, 0, s>>>(part_ml, part_o, n_rows, n_splits, hd, (bf16*)out);
        MLC_LAUNCH_CHECK();
    }
    return 0;
}

// The allocation-free variant of the split-key attention; see attention_noalloc.h for who
// it is for, what it costs and what a caller must keep in mind.
//
// It runs the very launch function of attention_simt.cu (included below for its kernels and
// that function, not for its entry points) and differs in one thing: the partial results go
// to the array `noalloc_scratch` of this file instead of caller-provided memory.
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
    if (hd <= 0 || q_heads <= 0 || n_splits < 1) return MLC_ERR_BAD_SIZE;
    float* part_ml = nullptr;
    float* part_o = nullptr;
    if (n_splits > 1) {                       // one split leaves no partial results: the array is not touched
        const long long rows = (long long)n_tokens * q_heads * n_splits;
        if (rows * (hd + 2) > (long long)MLC_NOALLOC_SCRATCH_FLOATS) return MLC_ERR_BAD_SIZE;   // beyond the fixed array: refuse
        float* scratch = nullptr;
        const int rc = scratch_address(&scratch);
        if (rc != 0) return rc;
        part_ml = scratch;                    // rows * 2 floats
        part_o = scratch + rows * 2;          // rows * hd floats
    }
    // the same checks, plan and kernels as the ordinary entry point (attention_simt.cu)
    return launch_attention_simt(q, out, dtype, cu_seqlens, start_pos, n_seqs, n_tokens, max_q_len, q_heads, kv_heads, hd,
                                 scale, window, n_splits, part_ml, part_o, k_pool, v_pool, page_table, entry_offset,
                                 pages_per_seq, page_size, (cudaStream_t)stream);
}

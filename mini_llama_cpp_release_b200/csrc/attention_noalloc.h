// Split-key attention over the paged cache for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project: the reference allocates a
// fresh device buffer for every intermediate result (src/cuda_tensor.cpp:57-63) and never
// splits a sequence's keys over blocks.
//
// Who needs it.  Splitting one sequence's keys over several blocks leaves partial results
// (a running maximum, a sum and a weighted value vector per row and split) that a second
// kernel merges.  The ordinary entry point, mlc_attention_simt, takes that scratch memory
// from its caller, who normally gets it from an allocator.  Some callers have no allocator
// they may use at the moment of the call: code embedded in another runtime that has handed
// all device memory to its own pool, so that cudaMalloc would fail or fight that pool; a
// serving loop that must not take the device-wide synchronisation cudaMalloc and cudaFree
// imply; a plain C program that links this library without PyTorch.  For them the scratch
// lives inside the library, in one fixed array in device memory.
//
// What it costs and where its limit is.  The array is
// MLC_NOALLOC_SCRATCH_FLOATS floats (4 MiB) and is part of the loaded library image: every
// GPU on which a process loads this library holds those 4 MiB until the process exits.  A
// call with n_splits > 1 needs n_tokens * q_heads * n_splits * (head_dim + 2) floats of it; a
// call that needs more is refused with MLC_ERR_BAD_SIZE (-2) and launches nothing.  A call
// with n_splits == 1 leaves no partial results, uses none of the array and has no such limit.
//
// What the caller must know.
//   * The first call on each device looks the array's device address up (the name of the
//     array in host code is only a handle, not an address a kernel could use) and remembers
//     it; make that first call outside any stream capture.
//   * All calls share the one array, and the array keeps whatever the previous call left.
//     That is harmless within a call: every element the merging kernel reads is written by
//     the same call's first kernel before, so nothing has to start at zero and nothing is
//     cleared.  But two calls that are in flight on the GPU at the same time (different
//     streams, or different threads) would write over each other's partial results: run the
//     calls on one stream, or otherwise order them.
//   * Inputs and outputs are the caller's, exactly as for mlc_attention_simt (same argument
//     meanings, same element types 0 = float32, 1 = bfloat16, same return convention); the
//     entry point calls no allocating routine of CUDA, of PyTorch or of any other library.
#pragma once

#define MLC_NOALLOC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int mlc_attention_split_noalloc(const void* q, void* out, int dtype, const int* cu_seqlens, const int* start_pos,
                                int n_seqs, int n_tokens, int max_q_len, int q_heads, int kv_heads, int head_dim,
                                float scale, int window, int n_splits, void* k_pool, void* v_pool,
                                const int* page_table, long long entry_offset, int pages_per_seq, int page_size,
                                void* stream);

#ifdef __cplusplus
}
#endif

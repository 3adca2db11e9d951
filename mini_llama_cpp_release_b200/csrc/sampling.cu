// Token selection on the device: argmax, temperature sampling and top-k sampling over
// float32 logits [rows][vocab], one block per row.
//
// Meanings are the reference sampler's (src/sampler.cpp:38-152; src/ops.cpp:179-192):
//   greedy     first index of the strict maximum (lowest id wins ties);
//   temperature  weight_i = exp((l_i - max)/T) over all ids in index order; draw r in
//              [0,1); the first i whose running sum of weight/total reaches r, else the last;
//   top-k      candidates sorted by logit descending, lower id first on ties, the first k
//              kept (k clamped to the vocabulary), then the same walk in that order.
// The reference draws r from one mt19937 per sampler; here r is a hash of
// (seed, sequence id, position), so a sequence draws the same numbers whatever batch it
// rides in.  The same hash is computed on the host by sampling/rng.py.
#include "common.cuh"

namespace mlc {

constexpr int SAMPLE_THREADS = 1024;
constexpr int TOPK_MAX = 1024;

__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Uniform float in [0, 1) with 24 random bits.
__host__ __device__ __forceinline__ float uniform_of(unsigned long long seed, int seq_id, int position) {
    unsigned long long h = mix64(seed);
    h = mix64(h ^ (unsigned long long)(unsigned int)seq_id);
    h = mix64(h ^ (unsigned long long)(unsigned int)position);
    return (float)(h >> 40) * (1.0f / 16777216.0f);
}

struct MaxIdx {
    float v;
    int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ MaxIdx block_argmax(MaxIdx v, MaxIdx* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx t;
        t.v = __shfl_xor_sync(0xffffffffu, v.v, o);
        t.i = __shfl_xor_sync(0xffffffffu, v.i, o);
        v = better(v, t);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int n_warps = (blockDim.x + 31) >> 5;
    MaxIdx t = (lane < n_warps) ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx u;
        u.v = __shfl_xor_sync(0xffffffffu, t.v, o);
        u.i = __shfl_xor_sync(0xffffffffu, t.i, o);
        t = better(t, u);
    }
    return t;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    __shared__ MaxIdx scratch[32];
    const float* row = logits + (long long)blockIdx.x * vocab;
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, MaxIdx{row[i], i});
    best = block_argmax(best, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = (best.i == 0x7fffffff) ? 0 : best.i;
}

// The same over many blocks per row: block (chunk, row) reduces its part of the row and leaves
// (value, index) in `partial`; the block that finishes a row last (counted in `done`, which it
// sets back to zero) merges the row's partial results.  `done` must be zero before the first call.
constexpr int ARGMAX_CHUNKS = 64;
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out, float* __restrict__ partial_v,
                    int* __restrict__ partial_i, unsigned int* __restrict__ done) {
    __shared__ MaxIdx scratch[32];
    __shared__ bool is_last;
    grid_launch_dependents();
    grid_dependency_wait();
    const int r = blockIdx.y, chunk = blockIdx.x;
    const float* row = logits + (long long)r * vocab;
    const int per = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int begin = chunk * per, end = min(vocab, begin + per);
    MaxIdx best{-INFINITY, 0x7fffffff};
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, MaxIdx{__ldg(row + i), i});
    best = block_argmax(best, scratch);
    if (threadIdx.x == 0) {
        partial_v[r * ARGMAX_CHUNKS + chunk] = best.v;
        partial_i[r * ARGMAX_CHUNKS + chunk] = best.i;
        __threadfence();
        is_last = atomicAdd(&done[r], 1u) == ARGMAX_CHUNKS - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    MaxIdx m{-INFINITY, 0x7fffffff};
    if (threadIdx.x < ARGMAX_CHUNKS) m = MaxIdx{partial_v[r * ARGMAX_CHUNKS + threadIdx.x], partial_i[r * ARGMAX_CHUNKS + threadIdx.x]};
    m = block_argmax(m, scratch);
    if (threadIdx.x == 0) {
        out[r] = (m.i == 0x7fffffff) ? 0 : m.i;
        done[r] = 0;
    }
}

// Inclusive scan of one float per thread over the block; returns this thread's inclusive
// prefix, *total gets the block's sum.  scratch: 32 floats.
__device__ __forceinline__ float block_scan(float v, float* scratch, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += t;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = x;
    __syncthreads();
    const int n_warps = (blockDim.x + 31) >> 5;
    float w = (lane < n_warps) ? scratch[lane] : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
    }
    const float before = (warp > 0) ? __shfl_sync(0xffffffffu, w, warp - 1) : 0.0f;
    *total = __shfl_sync(0xffffffffu, w, n_warps - 1);
    return x + before;
}

__device__ __forceinline__ int block_scan_int(int v, int* scratch, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += t;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = x;
    __syncthreads();
    const int n_warps = (blockDim.x + 31) >> 5;
    int w = (lane < n_warps) ? scratch[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
    }
    const int before = (warp > 0) ? __shfl_sync(0xffffffffu, w, warp - 1) : 0;
    *total = __shfl_sync(0xffffffffu, w, n_warps - 1);
    return x + before;
}

// Temperature sampling over the whole vocabulary in index order.  Each thread owns a
// contiguous run of ids so that prefix sums follow the index order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_temperature_kernel(const float* __restrict__ logits, int vocab, float temperature,
                          unsigned long long seed, const unsigned long long* __restrict__ seed_ptr, const int* __restrict__ seq_ids,
                          const int* __restrict__ positions, int* __restrict__ out) {
    __shared__ float fscratch[32];
    __shared__ int first_thread;
    const float* row = logits + (long long)blockIdx.x * vocab;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, fscratch);

    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * per), end = min(vocab, begin + per);
    float mine = 0.0f;
    for (int i = begin; i < end; ++i) mine += expf((row[i] - mx) / temperature);
    float total;
    const float incl = block_scan(mine, fscratch, &total);
    const float r = uniform_of(seed_ptr != nullptr ? *seed_ptr : seed, seq_ids[blockIdx.x], positions[blockIdx.x]);
    const float target = r * total;
    if (threadIdx.x == 0) first_thread = 0x7fffffff;
    __syncthreads();
    if (end > begin && incl >= target) atomicMin(&first_thread, (int)threadIdx.x);
    __syncthreads();
    if (first_thread == 0x7fffffff) {
        if (threadIdx.x == 0) out[blockIdx.x] = vocab - 1;
        return;
    }
    if ((int)threadIdx.x == first_thread) {
        float cum = incl - mine;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            cum += expf((row[i] - mx) / temperature);
            if (cum >= target) {
                pick = i;
                break;
            }
        }
        out[blockIdx.x] = pick;
    }
}

// Order-preserving map float → unsigned: larger float, larger key.
__device__ __forceinline__ unsigned int float_key(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Top-k sampling: radix-select the k-th largest key, gather the candidates (ties at the
// threshold by lowest id), sort them by (logit descending, id ascending), walk.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_top_k_kernel(const float* __restrict__ logits, int vocab, float temperature, int top_k,
                    unsigned long long seed, const unsigned long long* __restrict__ seed_ptr, const int* __restrict__ seq_ids,
                    const int* __restrict__ positions, int* __restrict__ out) {
    __shared__ unsigned int hist[256];
    __shared__ float cand_v[TOPK_MAX];
    __shared__ int cand_i[TOPK_MAX];
    __shared__ float fscratch[32];
    __shared__ int iscratch[32];
    __shared__ unsigned int sh_prefix;
    __shared__ int sh_remaining, n_greater, first_slot;

    const float* row = logits + (long long)blockIdx.x * vocab;
    const int k = min(top_k, vocab);

    // --- the k-th largest key, 8 bits at a time from the top
    unsigned int prefix = 0, mask = 0;
    int remaining = k;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned int key = float_key(row[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int rem = remaining;
            int digit = 255;
            for (; digit > 0; --digit) {
                const int cnt = (int)hist[digit];
                if (cnt >= rem) break;
                rem -= cnt;
            }
            sh_prefix = prefix | ((unsigned int)digit << shift);
            sh_remaining = rem;
        }
        __syncthreads();
        prefix = sh_prefix;
        remaining = sh_remaining;
        mask |= 255u << shift;
        __syncthreads();
    }
    const unsigned int thr = prefix;          // key of the k-th largest
    const int need_equal = remaining;         // how many ids equal to it are kept (lowest first)

    // --- gather: keys above the threshold in any order, keys equal to it in id order
    if (threadIdx.x == 0) n_greater = 0;
    __syncthreads();
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, (int)threadIdx.x * per), end = min(vocab, begin + per);
    int my_equal = 0;
    for (int i = begin; i < end; ++i) {
        const unsigned int key = float_key(row[i]);
        if (key > thr) {
            const int slot = atomicAdd(&n_greater, 1);
            cand_v[slot] = row[i];
            cand_i[slot] = i;
        } else if (key == thr) {
            ++my_equal;
        }
    }
    int total_equal;
    const int incl_equal = block_scan_int(my_equal, iscratch, &total_equal);
    __syncthreads();
    int rank = incl_equal - my_equal;          // equal ids before this thread's run
    const int base = n_greater;                // = k - need_equal
    for (int i = begin; i < end && rank < need_equal; ++i) {
        if (float_key(row[i]) == thr) {
            cand_v[base + rank] = row[i];
            cand_i[base + rank] = i;
            ++rank;
        }
    }
    __syncthreads();

    // --- pad to a power of two and sort by (value descending, id ascending)
    int n_sort = 1;
    while (n_sort < k) n_sort <<= 1;
    for (int i = k + threadIdx.x; i < n_sort; i += blockDim.x) {
        cand_v[i] = -INFINITY;
        cand_i[i] = 0x7fffffff;
    }
    __syncthreads();
    for (int size = 2; size <= n_sort; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = threadIdx.x; t < n_sort / 2; t += blockDim.x) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool descending_block = ((lo & size) == 0);
                const float va = cand_v[lo], vb = cand_v[hi];
                const int ia = cand_i[lo], ib = cand_i[hi];
                const bool a_first = (va > vb) || (va == vb && ia < ib);   // a belongs before b
                if (a_first != descending_block) {
                    cand_v[lo] = vb; cand_v[hi] = va;
                    cand_i[lo] = ib; cand_i[hi] = ia;
                }
            }
            __syncthreads();
        }
    }

    // --- weights, running sum in sorted order, first slot that reaches r
    const float mx = cand_v[0];
    const int t = threadIdx.x;
    const float w = (t < k) ? expf((cand_v[t] - mx) / temperature) : 0.0f;
    float total;
    const float incl = block_scan(w, fscratch, &total);
    const float r = uniform_of(seed_ptr != nullptr ? *seed_ptr : seed, seq_ids[blockIdx.x], positions[blockIdx.x]);
    const float target = r * total;
    if (threadIdx.x == 0) first_slot = k - 1;
    __syncthreads();
    if (t < k && incl >= target) atomicMin(&first_slot, t);
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = cand_i[first_slot];
}

}  // namespace mlc

using namespace mlc;

extern "C" int mlc_argmax(const float* logits, int rows, int vocab, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) return MLC_ERR_BAD_SIZE;
    argmax_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, out);
    MLC_LAUNCH_CHECK();
    return 0;
}

// temperature > 0.  top_k == 0: the whole vocabulary in index order; 2 <= top_k <= 1024 (after
// clamping to the vocabulary): sorted candidates.  Greedy cases go to mlc_argmax.
// scratch: rows * 64 floats, rows * 64 ints and rows counters that are zero (they are left zero).
extern "C" int mlc_argmax_split(const float* logits, int rows, int vocab, int* out, float* partial_v, int* partial_i,
                                unsigned int* done, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || rows > 65535) return MLC_ERR_BAD_SIZE;
    cudaError_t e = launch_pdl(argmax_split_kernel, dim3(ARGMAX_CHUNKS, rows), dim3(256), 0, (cudaStream_t)stream, logits, vocab, out,
                               partial_v, partial_i, done);
    return e == cudaSuccess ? 0 : (int)e;
}

// seed_ptr: null, or where on the device the seed stands (8-byte aligned): it is then read at every launch, so a
// captured launch serves any seed.
extern "C" int mlc_sample(const float* logits, int rows, int vocab, float temperature, int top_k,
                          unsigned long long seed, const unsigned long long* seed_ptr, const int* seq_ids,
                          const int* positions, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || !(temperature > 0.0f) || top_k < 0 || top_k == 1) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (top_k == 0) {
        sample_temperature_kernel<<<rows, SAMPLE_THREADS, 0, s>>>(logits, vocab, temperature, seed, seed_ptr, seq_ids,
                                                                  positions, out);
    } else {
        const int k = top_k < vocab ? top_k : vocab;
        if (k > TOPK_MAX) return MLC_ERR_UNSUPPORTED;
        sample_top_k_kernel<<<rows, SAMPLE_THREADS, 0, s>>>(logits, vocab, temperature, top_k, seed, seed_ptr, seq_ids,
                                                            positions, out);
    }
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" float mlc_uniform_of(unsigned long long seed, int seq_id, int position) {
    return uniform_of(seed, seq_id, position);
}

// After a decode step whose tokens were chosen on the device: make the chosen tokens the
// next step's input and move every sequence one position on, so that the next step can
// start without the host.  `history`, if given, keeps each step's choices
// [max_steps][n]; `counter` counts the steps taken.
__global__ void decode_advance_kernel(const int* __restrict__ chosen, int n, int* __restrict__ tokens,
                                      int* __restrict__ positions, int* __restrict__ start_pos,
                                      int* __restrict__ sample_pos, int* __restrict__ history,
                                      int* __restrict__ counter, int max_steps) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int step = *counter;
    if (i < n) {
        tokens[i] = chosen[i];
        positions[i] += 1;
        start_pos[i] += 1;
        sample_pos[i] += 1;
        if (history != nullptr && step < max_steps) history[(long long)step * n + i] = chosen[i];
    }
    __syncthreads();
    if (i == 0) *counter = step + 1;
}

extern "C" int mlc_decode_advance(const int* chosen, int n, int* tokens, int* positions, int* start_pos,
                                  int* sample_pos, int* history, int* counter, int max_steps, void* stream) {
    if (n <= 0) return 0;
    if (n > 1024) return MLC_ERR_BAD_SIZE;
    cudaError_t e = mlc::launch_pdl(decode_advance_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, chosen, n, tokens,
                                    positions, start_pos, sample_pos, history, counter, max_steps);
    return e == cudaSuccess ? 0 : (int)e;
}

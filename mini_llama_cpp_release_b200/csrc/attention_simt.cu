// Attention over the paged cache in plain float32 arithmetic (no tensor cores), for any
// element type of the cache and any head size up to 256.  It is the whole-model 32-bit
// path's attention and the yardstick the tensor-core kernels are checked against.
//
// One kernel serves prompts, continuation chunks and single decoded tokens: a step gives
// each sequence q_len new tokens at positions start_pos .. start_pos + q_len - 1, their
// keys and values are already in the cache, and a token at position p reads keys
// lo(p) .. p, with lo(p) = 0 or p - window + 1.  The reference computes the same thing
// one (head, position) at a time: score = (q·k)·1/sqrt(hd), max, exp, sum, weighted sum
// of values (src/forward.cpp:585-611; src/ops.cpp:43-70); query head h reads kv head
// h / (H/KV) (src/forward.cpp:524-526).  Here a block holds up to 16 (token, head) rows
// that share one kv head, streams 32-key tiles through shared memory and keeps a running
// maximum and sum per row; long key ranges can be split over blocks, whose partial
// (max, sum, weighted values) are merged by a second kernel.
#include "common.cuh"

namespace mlc {

constexpr int ATT_ROWS = 16;       // (token, head) rows per block
constexpr int ATT_WARPS = 4;
constexpr int ATT_ROWS_PER_WARP = ATT_ROWS / ATT_WARPS;
constexpr int ATT_TILE = 32;       // keys per tile: one per lane
constexpr int ATT_MAX_HD = 256;
constexpr int ATT_ACC = ATT_MAX_HD / 32;

struct AttnArgs {
    const void* q;            // [N][H][hd]
    void* out;                // [N][H][hd]
    const int* cu_seqlens;    // [B+1] token offsets of this step
    const int* start_pos;     // [B] tokens cached before this step
    float* part_ml;           // [N*H][n_splits][2]   (n_splits > 1)
    float* part_o;            // [N*H][n_splits][hd]
    float scale;
    int q_heads;
    int group;                // query heads per kv head
    int window;               // 0: all keys
    int tokens_per_block;     // TQ
    int heads_per_block;      // GH, TQ*GH <= 16
    int head_chunks;          // ceil(group / GH)
    int n_splits;
};

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_simt_kernel(AttnArgs a, PagedKV c) {
    extern __shared__ float smem[];
    const int hd = c.head_dim;
    float* Qs = smem;                              // [16][hd]
    float* Ks = Qs + ATT_ROWS * hd;                // [32][hd+1]
    float* Vs = Ks + ATT_TILE * (hd + 1);          // [32][hd]
    __shared__ long long key_off[ATT_TILE];

    const int b = blockIdx.z;
    int y = blockIdx.y;
    const int split = y % a.n_splits;  y /= a.n_splits;
    const int chunk = y % a.head_chunks;  y /= a.head_chunks;
    const int kvh = y;
    const int tok0 = blockIdx.x * a.tokens_per_block;
    const int seq_tok0 = a.cu_seqlens[b];
    const int q_len = a.cu_seqlens[b + 1] - seq_tok0;
    if (tok0 >= q_len) return;
    const int start = a.start_pos[b];
    const int n_tok = min(a.tokens_per_block, q_len - tok0);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* q = (const T*)a.q;

    // stage the block's query rows
    for (int idx = threadIdx.x; idx < ATT_ROWS * hd; idx += blockDim.x) {
        const int r = idx / hd, d = idx % hd;
        const int t = r / a.heads_per_block, hg = chunk * a.heads_per_block + r % a.heads_per_block;
        float v = 0.0f;
        if (t < n_tok && hg < a.group) {
            const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
            v = to_float(q[row * hd + d]);
        }
        Qs[idx] = v;
    }

    // key range of the block and of this split
    const int p_first = start + tok0, p_last = start + tok0 + n_tok - 1;
    const int lo_block = (a.window > 0) ? max(0, p_first - a.window + 1) : 0;
    const int tile_begin = lo_block / ATT_TILE, tile_end = p_last / ATT_TILE + 1;
    const int per_split = (tile_end - tile_begin + a.n_splits - 1) / a.n_splits;
    const int my_begin = tile_begin + split * per_split;
    const int my_end = min(tile_end, my_begin + per_split);

    float m[ATT_ROWS_PER_WARP], l[ATT_ROWS_PER_WARP], acc[ATT_ROWS_PER_WARP][ATT_ACC];
    int row_lo[ATT_ROWS_PER_WARP], row_hi[ATT_ROWS_PER_WARP];
    bool row_ok[ATT_ROWS_PER_WARP];
#pragma unroll
    for (int i = 0; i < ATT_ROWS_PER_WARP; ++i) {
        const int r = warp * ATT_ROWS_PER_WARP + i;
        const int t = r / a.heads_per_block, hg = chunk * a.heads_per_block + r % a.heads_per_block;
        row_ok[i] = (t < n_tok) && (hg < a.group);
        row_hi[i] = start + tok0 + t;
        row_lo[i] = (a.window > 0) ? max(0, row_hi[i] - a.window + 1) : 0;
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int k = 0; k < ATT_ACC; ++k) acc[i][k] = 0.0f;
    }

    const T* kp = (const T*)c.k_pool;
    const T* vp = (const T*)c.v_pool;
    for (int tile = my_begin; tile < my_end; ++tile) {
        __syncthreads();   // previous tile's readers are done (and Qs is staged)
        if (threadIdx.x < ATT_TILE) {
            const int kpos = tile * ATT_TILE + threadIdx.x;
            key_off[threadIdx.x] = (kpos >= lo_block && kpos <= p_last) ? paged_offset(c, b, kpos, kvh) : -1;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < ATT_TILE * hd; idx += blockDim.x) {
            const int j = idx / hd, d = idx % hd;
            const long long off = key_off[j];
            float kv = 0.0f, vv = 0.0f;
            if (off >= 0) {
                kv = to_float(kp[off + d]);
                vv = to_float(vp[off + d]);
            }
            Ks[j * (hd + 1) + d] = kv;
            Vs[j * hd + d] = vv;
        }
        __syncthreads();

        const int kpos = tile * ATT_TILE + lane;
#pragma unroll
        for (int i = 0; i < ATT_ROWS_PER_WARP; ++i) {
            if (!row_ok[i]) continue;
            const bool in_range = kpos >= row_lo[i] && kpos <= row_hi[i];
            float s = -INFINITY;
            if (in_range) {
                const float* qr = Qs + (warp * ATT_ROWS_PER_WARP + i) * hd;
                const float* kr = Ks + lane * (hd + 1);
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot += qr[d] * kr[d];
                s = dot * a.scale;
            }
            const float tile_max = warp_max(s);
            if (tile_max == -INFINITY) continue;
            const float m_new = fmaxf(m[i], tile_max);
            const float p = in_range ? expf(s - m_new) : 0.0f;
            const float corr = (m[i] == -INFINITY) ? 0.0f : expf(m[i] - m_new);
            l[i] = l[i] * corr + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int k = 0; k < ATT_ACC; ++k) acc[i][k] *= corr;
            for (int j = 0; j < ATT_TILE; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                const float* vr = Vs + j * hd;
#pragma unroll
                for (int k = 0; k < ATT_ACC; ++k) {
                    const int d = lane + 32 * k;
                    if (d < hd) acc[i][k] += pj * vr[d];
                }
            }
        }
    }

    // results
#pragma unroll
    for (int i = 0; i < ATT_ROWS_PER_WARP; ++i) {
        if (!row_ok[i]) continue;
        const int r = warp * ATT_ROWS_PER_WARP + i;
        const int t = r / a.heads_per_block, hg = chunk * a.heads_per_block + r % a.heads_per_block;
        const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
        if (a.n_splits == 1) {
            T* o = (T*)a.out + row * hd;
            const float inv = 1.0f / l[i];
#pragma unroll
            for (int k = 0; k < ATT_ACC; ++k) {
                const int d = lane + 32 * k;
                if (d < hd) o[d] = from_float<T>(acc[i][k] * inv);
            }
        } else {
            const long long pr = row * a.n_splits + split;
            if (lane == 0) {
                a.part_ml[pr * 2] = m[i];
                a.part_ml[pr * 2 + 1] = l[i];
            }
#pragma unroll
            for (int k = 0; k < ATT_ACC; ++k) {
                const int d = lane + 32 * k;
                if (d < hd) a.part_o[pr * hd + d] = acc[i][k];
            }
        }
    }
}

// Merge the partial results of the key splits of each (token, head) row; one warp per row.
// The lanes first share out the splits (maximum, weights, sum), then the output dims; the
// loads of a lane do not depend on each other, so they are in flight together.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_ml, const float* __restrict__ part_o,
                                         long long n_rows, int n_splits, int hd, T* __restrict__ out) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const float* ml = part_ml + row * n_splits * 2;
    float M = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, __ldg(ml + 2 * s));
    M = warp_max(M);
    float L = 0.0f;
    for (int s = lane; s < n_splits; s += 32) {
        const float ms = __ldg(ml + 2 * s);
        if (ms != -INFINITY) L += __ldg(ml + 2 * s + 1) * expf(ms - M);
    }
    L = warp_sum(L);
    const float inv = 1.0f / L;
    const float* po = part_o + row * n_splits * hd;
    for (int d = lane; d < hd; d += 32) {
        float o = 0.0f;
#pragma unroll 8
        for (int s = 0; s < n_splits; ++s) {
            const float ms = __ldg(ml + 2 * s);
            const float w = (ms != -INFINITY) ? expf(ms - M) : 0.0f;
            const float v = __ldg(po + (long long)s * hd + d);
            o += (w != 0.0f) ? v * w : 0.0f;           // an empty split's values were never written
        }
        out[row * hd + d] = from_float<T>(o * inv);
    }
}

}  // namespace mlc

// The launch shared by every entry point of the split-key attention (the ordinary one below and the one that keeps
// its scratch inside the library): checks, the plan of heads and tokens per block, the two kernels.
// n_splits > 1 needs part_ml (n_tokens*q_heads*n_splits*2 floats) and part_o (n_tokens*q_heads*n_splits*hd).
namespace mlc {
static int launch_attention_simt(const void* q, void* out, int dtype, const int* cu_seqlens, const int* start_pos,
                                 int n_seqs, int n_tokens, int max_q_len, int q_heads, int kv_heads, int hd, float scale,
                                 int window, int n_splits, float* part_ml, float* part_o, void* k_pool, void* v_pool,
                                 const int* page_table, long long entry_offset, int pages_per_seq, int page_size,
                                 cudaStream_t s) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (hd <= 0 || hd > ATT_MAX_HD || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return MLC_ERR_BAD_SIZE;
    if (n_splits < 1 || (n_splits > 1 && (part_ml == nullptr || part_o == nullptr))) return MLC_ERR_BAD_SIZE;
    if (n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    if (dtype != MLC_DTYPE_F32 && dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
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
    cudaError_t e;
    if (dtype == MLC_DTYPE_F32) {
        static size_t allowed_f32 = 48 * 1024;
        if (smem > allowed_f32) {
            e = cudaFuncSetAttribute(attention_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            allowed_f32 = smem;
        }
        attention_simt_kernel<float><<<grid, ATT_WARPS * 32, smem, s>>>(a, c);
    } else {
        static size_t allowed_bf16 = 48 * 1024;
        if (smem > allowed_bf16) {
            e = cudaFuncSetAttribute(attention_simt_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            allowed_bf16 = smem;
        }
        attention_simt_kernel<bf16><<<grid, ATT_WARPS * 32, smem, s>>>(a, c);
    }
    MLC_LAUNCH_CHECK();
    // With one split the first kernel has written `out` itself and no scratch was touched; with more, every
    // (row, split) pair of the scratch was written above before the merge reads it.
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
}  // namespace mlc

#ifndef MLC_KERNELS_ONLY   // a file that includes this one for its kernels defines its own entry points
using namespace mlc;

// q, out: [n_tokens][q_heads][hd] of `dtype`; the cache pools hold the same type.
// max_q_len: the longest sequence of this step (sizes the grid).  n_splits > 1 needs
// part_ml (n_tokens*q_heads*n_splits*2 floats) and part_o (n_tokens*q_heads*n_splits*hd).
extern "C" int mlc_attention_simt(const void* q, void* out, int dtype, const int* cu_seqlens,
                                  const int* start_pos, int n_seqs, int n_tokens, int max_q_len, int q_heads,
                                  int kv_heads, int hd, float scale, int window, int n_splits, float* part_ml,
                                  float* part_o, void* k_pool, void* v_pool, const int* page_table,
                                  long long entry_offset, int pages_per_seq, int page_size, void* stream) {
    return launch_attention_simt(q, out, dtype, cu_seqlens, start_pos, n_seqs, n_tokens, max_q_len, q_heads, kv_heads, hd,
                                 scale, window, n_splits, part_ml, part_o, k_pool, v_pool, page_table, entry_offset,
                                 pages_per_seq, page_size, (cudaStream_t)stream);
}

// Merge partial results that another attention kernel left in part_ml / part_o
// (maxima in natural-log units, sums and weighted values relative to them).
extern "C" int mlc_attention_combine(const float* part_ml, const float* part_o, long long n_rows, int n_splits,
                                     int hd, void* out, int dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (n_splits < 1 || hd <= 0) return MLC_ERR_BAD_SIZE;
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == MLC_DTYPE_F32)
        e = launch_pdl(attention_combine_kernel<float>, dim3(blocks), dim3(128), 0, s, part_ml, part_o, n_rows, n_splits, hd, (float*)out);
    else if (dtype == MLC_DTYPE_BF16)
        e = launch_pdl(attention_combine_kernel<bf16>, dim3(blocks), dim3(128), 0, s, part_ml, part_o, n_rows, n_splits, hd, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    return e == cudaSuccess ? 0 : (int)e;
}
#endif  // MLC_KERNELS_ONLY

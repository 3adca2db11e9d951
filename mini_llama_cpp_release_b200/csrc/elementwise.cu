// Row-wise kernels around the matrix products: embedding gather, residual add fused with
// RMSNorm, the rotation table, the Q/K/V epilogue (bias, rotate-half RoPE, scatter of keys
// and values into the paged cache), SiLU(gate)·up, and row gather.
//
// The arithmetic follows the reference's scalar code and stays in float32 wherever the
// reference's does: the sum of squares and 1/sqrt(ss/d + eps) with the multiply order
// x·scale·w (src/ops.cpp:19-41), cos/sin of a float32 angle p·f_i and the pairing
// (i, i + hd/2) (src/ops.cpp:125-141), gate·(1/(1+exp(-gate)))·up (src/ops.cpp:94-107),
// the residual sum (src/forward.cpp:772, 779).  What is new is the fusion and the layout.
#include "common.cuh"

namespace mlc {

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, int d,
                             float* __restrict__ out) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int n = blockIdx.x;
    const T* row = table + (long long)ids[n] * d;
    float* o = out + (long long)n * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(row[i]);
}

// ------------------------------------------------------------------ residual add + RMSNorm
// x (float32, the residual stream) += the sum of the delta slices, when given (a branch output,
// possibly left as split-K partial sums [n_slices][n][d]); out = x·scale·gain.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_slices,
                                   long long slice_stride, const float* __restrict__ gain, float eps, int d,
                                   T* __restrict__ out) {
    __shared__ float scratch[32];
    grid_launch_dependents();
    grid_dependency_wait();
    const long long base = (long long)blockIdx.x * d;
    float ss = 0.0f;
    if (delta != nullptr) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = x[base + i];
#pragma unroll 8
            for (int s = 0; s < n_slices; ++s) v += __ldg(delta + s * slice_stride + base + i);
            x[base + i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = x[base + i];
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        out[base + i] = from_float<T>(x[base + i] * scale * gain[i]);
    }
}

// The same with 16-byte accesses, for rows whose length is a multiple of 4 (all pointers 16-byte aligned).
template <typename T>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_slices,
                                        long long slice_stride, const float* __restrict__ gain, float eps, int d,
                                        T* __restrict__ out) {
    __shared__ float scratch[32];
    grid_launch_dependents();
    grid_dependency_wait();
    const long long base = (long long)blockIdx.x * d;
    const int d4 = d >> 2;
    float4* x4 = reinterpret_cast<float4*>(x + base);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        float4 v = x4[i];
        if (delta != nullptr) {
#pragma unroll 4
            for (int s = 0; s < n_slices; ++s) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(delta + s * slice_stride + base) + i);
                v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            }
            x4[i] = v;
        }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 v = x4[i], g = __ldg(g4 + i);
        T* o = out + base + 4 * i;
        o[0] = from_float<T>(v.x * scale * g.x);
        o[1] = from_float<T>(v.y * scale * g.y);
        o[2] = from_float<T>(v.z * scale * g.z);
        o[3] = from_float<T>(v.w * scale * g.w);
    }
}

// Many rows (prompts): one warp per row, the row held in registers between the sum of squares and the scaling, so
// that every element is read once and the loads of a row are all in flight together; no block-wide barrier.
// NV = 16-byte pieces per lane (d <= 128 * NV).
template <typename T, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_slices, long long slice_stride,
                        const float* __restrict__ gain, float eps, int d, int n, T* __restrict__ out) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const long long base = (long long)row * d;
    const int d4 = d >> 2;
    float4* x4 = reinterpret_cast<float4*>(x + base);
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane + 32 * k;
        v[k] = (i < d4) ? x4[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (delta != nullptr) {
        for (int s = 0; s < n_slices; ++s) {
            const float4* t4 = reinterpret_cast<const float4*>(delta + s * slice_stride + base);
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int i = lane + 32 * k;
                if (i < d4) {
                    const float4 t = __ldg(t4 + i);
                    v[k].x += t.x; v[k].y += t.y; v[k].z += t.z; v[k].w += t.w;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = lane + 32 * k;
            if (i < d4) x4[i] = v[k];
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    const float4* g4 = reinterpret_cast<const float4*>(gain);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = lane + 32 * k;
        if (i < d4) {
            const float4 g = __ldg(g4 + i);
            const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z, e = v[k].w * scale * g.w;
            if (sizeof(T) == 4) {
                reinterpret_cast<float4*>(out + base)[i] = make_float4(a, b, c, e);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
                reinterpret_cast<uint2*>(out + base)[i] = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
            }
        }
    }
}

template <typename T>
static cudaError_t launch_rmsnorm_warp(int nv, float* x, const float* delta, int n_slices, long long stride, const float* gain,
                                       float eps, int d, int n, T* out, cudaStream_t s) {
    const dim3 grid((n + 7) / 8), block(256);
    switch (nv) {
        case 1: return launch_pdl(add_rmsnorm_warp_kernel<T, 1>, grid, block, 0, s, x, delta, n_slices, stride, gain, eps, d, n, out);
        case 2: return launch_pdl(add_rmsnorm_warp_kernel<T, 2>, grid, block, 0, s, x, delta, n_slices, stride, gain, eps, d, n, out);
        case 3: case 4: return launch_pdl(add_rmsnorm_warp_kernel<T, 4>, grid, block, 0, s, x, delta, n_slices, stride, gain, eps, d, n, out);
        case 5: case 6: case 7: case 8:
            return launch_pdl(add_rmsnorm_warp_kernel<T, 8>, grid, block, 0, s, x, delta, n_slices, stride, gain, eps, d, n, out);
        default: return launch_pdl(add_rmsnorm_warp_kernel<T, 16>, grid, block, 0, s, x, delta, n_slices, stride, gain, eps, d, n, out);
    }
}

// ------------------------------------------------------------------ rotation table
// table[p][i] = (cos(p·f_i), sin(p·f_i)), the angle formed in float32 from an integer
// position and a float32 frequency, as src/ops.cpp:132-134 does for each token.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int n_pos, int half,
                                  float2* __restrict__ table) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_pos * half) return;
    const int p = (int)(idx / half), i = (int)(idx % half);
    const float angle = (float)p * inv_freq[i];
    table[idx] = make_float2(cosf(angle), sinf(angle));
}

// ------------------------------------------------------------------ Q/K/V epilogue
// One block per token.  Input row: [q heads | k heads | v heads] in float32 straight from
// the projection.  Adds the bias, rotates q and k by the token's position, writes q as
// [token][head][hd] in the activation type and k, v into the token's place in the cache.
// With kv_heads_in_row == 0 the row holds q only (a layer that reads another's cache).
template <typename T>
__global__ void qkv_post_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                                const int* __restrict__ positions, const int* __restrict__ tok_seq,
                                const float2* __restrict__ rope, int rope_positions, int q_heads,
                                int kv_heads_in_row, int hd, T* __restrict__ q_out, PagedKV cache) {
    const int n = blockIdx.x;
    const int half = hd >> 1;
    const int row_width = (q_heads + 2 * kv_heads_in_row) * hd;
    const float* row = qkv + (long long)n * row_width;
    const int p = positions[n];
    const int seq = tok_seq[n];
    const float2* cs = (rope != nullptr) ? rope + (long long)min(p, rope_positions - 1) * half : nullptr;

    // q and k heads: one thread per rotation pair
    const int rot_heads = q_heads + kv_heads_in_row;
    for (int idx = threadIdx.x; idx < rot_heads * half; idx += blockDim.x) {
        const int head = idx / half, i = idx % half;
        const int c0 = head * hd + i, c1 = c0 + half;
        float x0 = row[c0], x1 = row[c1];
        if (bias != nullptr) {
            x0 += bias[c0];
            x1 += bias[c1];
        }
        float y0 = x0, y1 = x1;
        if (cs != nullptr) {
            const float2 t = cs[i];
            y0 = x0 * t.x - x1 * t.y;
            y1 = x0 * t.y + x1 * t.x;
        }
        if (head < q_heads) {
            T* dst = q_out + ((long long)n * q_heads + head) * hd;
            dst[i] = from_float<T>(y0);
            dst[i + half] = from_float<T>(y1);
        } else {
            T* dst = (T*)cache.k_pool + paged_offset(cache, seq, p, head - q_heads);
            dst[i] = from_float<T>(y0);
            dst[i + half] = from_float<T>(y1);
        }
    }
    // v heads: bias only
    const int v_start = (q_heads + kv_heads_in_row) * hd;
    for (int idx = threadIdx.x; idx < kv_heads_in_row * hd; idx += blockDim.x) {
        const int head = idx / hd, i = idx % hd;
        float v = row[v_start + idx];
        if (bias != nullptr) v += bias[v_start + idx];
        T* dst = (T*)cache.v_pool + paged_offset(cache, seq, p, head);
        dst[i] = from_float<T>(v);
    }
}

// ------------------------------------------------------------------ SiLU(gate)·up
// Input row [gate (I) | up (I)], or with `interleaved` [g0, u0, g1, u1, ...]; output [I].
template <typename TIn, typename TOut>
__global__ void silu_mul_kernel(const TIn* __restrict__ gu, int inter, long long total, int interleaved,
                                TOut* __restrict__ out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long n = idx / inter;
    const int i = (int)(idx % inter);
    const TIn* row = gu + n * 2 * inter;
    const float g = to_float(interleaved ? row[2 * i] : row[i]);
    const float u = to_float(interleaved ? row[2 * i + 1] : row[inter + i]);
    const float sig = 1.0f / (1.0f + expf(-g));
    out[idx] = from_float<TOut>(g * sig * u);
}

// Eight outputs per thread with 16-byte loads and stores (bfloat16 in and out, I a multiple of 8).
__global__ void silu_mul_vec8_kernel(const bf16* __restrict__ gu, int inter, long long total_vec, int interleaved,
                                     bf16* __restrict__ out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_vec) return;
    const int per_row = inter >> 3;
    const long long n = idx / per_row;
    const int i = (int)(idx % per_row) << 3;
    const bf16* row = gu + n * 2 * inter;
    float g[8], u[8];
    if (interleaved) {
        const uint4 a = *reinterpret_cast<const uint4*>(row + 2 * i);
        const uint4 b = *reinterpret_cast<const uint4*>(row + 2 * i + 8);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 fa = __bfloat1622float2(pa[k]), fb = __bfloat1622float2(pb[k]);
            g[k] = fa.x; u[k] = fa.y;
            g[4 + k] = fb.x; u[4 + k] = fb.y;
        }
    } else {
        const uint4 a = *reinterpret_cast<const uint4*>(row + i);
        const uint4 b = *reinterpret_cast<const uint4*>(row + inter + i);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 fa = __bfloat1622float2(pa[k]), fb = __bfloat1622float2(pb[k]);
            g[2 * k] = fa.x; g[2 * k + 1] = fa.y;
            u[2 * k] = fb.x; u[2 * k + 1] = fb.y;
        }
    }
    uint4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float y0 = g[2 * k] * (1.0f / (1.0f + expf(-g[2 * k]))) * u[2 * k];
        const float y1 = g[2 * k + 1] * (1.0f / (1.0f + expf(-g[2 * k + 1]))) * u[2 * k + 1];
        po[k] = __floats2bfloat162_rn(y0, y1);
    }
    *reinterpret_cast<uint4*>(out + n * inter + i) = o;
}

// ------------------------------------------------------------------ row gather
__global__ void gather_rows_kernel(const float* __restrict__ x, const float* __restrict__ delta, int n_slices,
                                   long long slice_stride, const int* __restrict__ rows, int d,
                                   float* __restrict__ out_x, float* __restrict__ out_delta) {
    grid_launch_dependents();
    grid_dependency_wait();
    const long long src = (long long)rows[blockIdx.x] * d, dst = (long long)blockIdx.x * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        out_x[dst + i] = x[src + i];
        if (delta != nullptr) {
            float v = 0.0f;
            for (int s = 0; s < n_slices; ++s) v += delta[s * slice_stride + src + i];
            out_delta[dst + i] = v;
        }
    }
}

// ------------------------------------------------------------------ dtype conversion
template <typename TIn, typename TOut>
__global__ void convert_kernel(const TIn* __restrict__ in, long long total, TOut* __restrict__ out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) out[idx] = from_float<TOut>(to_float(in[idx]));
}

static inline int row_threads(int d) {
    int t = 32;
    while (t < d && t < 256) t <<= 1;
    return t;
}

// Few rows: one element per thread where the row allows it, so that every load of the row is in flight at once.
static inline int norm_threads(int d, int n) {
    if (n > 1024) return row_threads(d);
    int t = 32;
    while (t < d && t < 1024) t <<= 1;
    return t;
}

}  // namespace mlc

using namespace mlc;

extern "C" int mlc_embed(const void* table, int table_dtype, const int* ids, int n, int d, float* out,
                         void* stream) {
    if (n <= 0) return 0;
    if (d <= 0) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e;
    if (table_dtype == MLC_DTYPE_F32)
        e = launch_pdl(embed_kernel<float>, dim3(n), dim3(norm_threads(d, n)), 0, s, (const float*)table, ids, d, out);
    else if (table_dtype == MLC_DTYPE_BF16)
        e = launch_pdl(embed_kernel<bf16>, dim3(n), dim3(norm_threads(d, n)), 0, s, (const bf16*)table, ids, d, out);
    else
        return MLC_ERR_BAD_DTYPE;
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int mlc_add_rmsnorm(float* x, const float* delta, int n_slices, const float* gain, float eps, int n, int d,
                               void* out, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || (delta != nullptr && n_slices < 1)) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long stride = (long long)n * d;
    cudaError_t e;
    const bool vec = (d & 3) == 0 && n > 64 &&
                     ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)gain) | ((uintptr_t)out)) & 15) == 0;
    const int nv = ((d >> 2) + 31) / 32;                 // 16-byte pieces per lane if a warp takes a row
    if (vec && nv <= 16 && n >= 256 && out_dtype == MLC_DTYPE_F32)
        e = launch_rmsnorm_warp<float>(nv, x, delta, n_slices, stride, gain, eps, d, n, (float*)out, s);
    else if (vec && nv <= 16 && n >= 256 && out_dtype == MLC_DTYPE_BF16)
        e = launch_rmsnorm_warp<bf16>(nv, x, delta, n_slices, stride, gain, eps, d, n, (bf16*)out, s);
    else if (vec && out_dtype == MLC_DTYPE_F32)
        e = launch_pdl(add_rmsnorm_vec4_kernel<float>, dim3(n), dim3(row_threads(d >> 2)), 0, s, x, delta, n_slices, stride, gain, eps, d, (float*)out);
    else if (vec && out_dtype == MLC_DTYPE_BF16)
        e = launch_pdl(add_rmsnorm_vec4_kernel<bf16>, dim3(n), dim3(row_threads(d >> 2)), 0, s, x, delta, n_slices, stride, gain, eps, d, (bf16*)out);
    else if (out_dtype == MLC_DTYPE_F32)
        e = launch_pdl(add_rmsnorm_kernel<float>, dim3(n), dim3(norm_threads(d, n)), 0, s, x, delta, n_slices, stride, gain, eps, d, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16)
        e = launch_pdl(add_rmsnorm_kernel<bf16>, dim3(n), dim3(norm_threads(d, n)), 0, s, x, delta, n_slices, stride, gain, eps, d, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    if (e != cudaSuccess) return (int)e;
    return 0;
}

extern "C" int mlc_rope_table(const float* inv_freq, int n_pos, int half, void* table, void* stream) {
    if (n_pos <= 0 || half <= 0) return MLC_ERR_BAD_SIZE;
    const long long total = (long long)n_pos * half;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(inv_freq, n_pos, half,
                                                                                         (float2*)table);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_qkv_post(const float* qkv, const float* bias, const int* positions, const int* tok_seq,
                            const void* rope_table, int rope_positions, int n, int q_heads,
                            int kv_heads_in_row, int hd, void* q_out, int dtype, void* k_pool, void* v_pool,
                            const int* page_table, long long entry_offset, int pages_per_seq, int page_size,
                            int cache_kv_heads, void* stream) {
    if (n <= 0) return 0;
    if (hd <= 0 || (hd & 1) || q_heads <= 0 || kv_heads_in_row < 0) return MLC_ERR_BAD_SIZE;
    if (kv_heads_in_row != 0 && kv_heads_in_row != cache_kv_heads) return MLC_ERR_BAD_SIZE;
    PagedKV c{k_pool, v_pool, page_table, entry_offset, pages_per_seq, page_size, cache_kv_heads, hd};
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = row_threads((q_heads + kv_heads_in_row) * hd / 2);
    if (dtype == MLC_DTYPE_F32)
        qkv_post_kernel<float><<<n, threads, 0, s>>>(qkv, bias, positions, tok_seq, (const float2*)rope_table,
                                                     rope_positions, q_heads, kv_heads_in_row, hd,
                                                     (float*)q_out, c);
    else if (dtype == MLC_DTYPE_BF16)
        qkv_post_kernel<bf16><<<n, threads, 0, s>>>(qkv, bias, positions, tok_seq, (const float2*)rope_table,
                                                    rope_positions, q_heads, kv_heads_in_row, hd, (bf16*)q_out,
                                                    c);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_silu_mul(const void* gate_up, int in_dtype, int n, int inter, int interleaved, void* out,
                            int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (inter <= 0) return MLC_ERR_BAD_SIZE;
    const long long total = (long long)n * inter;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_BF16 && (inter & 7) == 0 &&
        ((((uintptr_t)gate_up) | ((uintptr_t)out)) & 15) == 0) {
        const long long total_vec = total >> 3;
        silu_mul_vec8_kernel<<<(unsigned)((total_vec + 255) / 256), 256, 0, s>>>((const bf16*)gate_up, inter, total_vec,
                                                                                 interleaved, (bf16*)out);
        MLC_LAUNCH_CHECK();
        return 0;
    }
    if (in_dtype == MLC_DTYPE_F32 && out_dtype == MLC_DTYPE_F32)
        silu_mul_kernel<float, float><<<blocks, 256, 0, s>>>((const float*)gate_up, inter, total, interleaved, (float*)out);
    else if (in_dtype == MLC_DTYPE_F32 && out_dtype == MLC_DTYPE_BF16)
        silu_mul_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)gate_up, inter, total, interleaved, (bf16*)out);
    else if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_BF16)
        silu_mul_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((const bf16*)gate_up, inter, total, interleaved, (bf16*)out);
    else if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_F32)
        silu_mul_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)gate_up, inter, total, interleaved, (float*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_gather_rows(const float* x, const float* delta, int n_slices, long long slice_stride, const int* rows,
                               int n_rows, int d, float* out_x, float* out_delta, void* stream) {
    if (n_rows <= 0) return 0;
    cudaError_t e = launch_pdl(gather_rows_kernel, dim3(n_rows), dim3(norm_threads(d, n_rows)), 0, (cudaStream_t)stream, x, delta,
                               n_slices, slice_stride, rows, d, out_x, out_delta);
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int mlc_convert(const void* in, int in_dtype, long long total, void* out, int out_dtype, void* stream) {
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == MLC_DTYPE_F32 && out_dtype == MLC_DTYPE_BF16)
        convert_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)in, total, (bf16*)out);
    else if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_F32)
        convert_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)in, total, (float*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

// Switch programmatic dependent launch on (1, the default) or off (0) for this library's kernels.
extern "C" int mlc_set_pdl(int enabled) {
    mlc::pdl_enabled() = enabled ? 1 : 0;
    return 0;
}

// A copy between pinned host memory and the device on the given stream, for the few hundred bytes a decode step
// brings and takes: the call costs the host a third of what a tensor library's copy does.  direction 0: host to
// device, 1: device to host.
extern "C" int mlc_copy_async(void* dst, const void* src, long long bytes, int direction, void* stream) {
    if (bytes <= 0) return 0;
    if (dst == nullptr || src == nullptr || (direction != 0 && direction != 1)) return MLC_ERR_BAD_SIZE;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, direction == 0 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

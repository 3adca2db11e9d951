// y[M][N] = x[M][K] · W[N][K]ᵀ with float32 multiply-adds on the CUDA cores: the linear
// layer of the whole-model 32-bit path, and the fallback for operand types the
// tensor-core kernels do not take.  No tensor-core mode of any precision is involved.
//
// The reference's linear is y = W·x for one row x, W row-major [out, in]
// (src/matmul_optimized.cpp:40-54, 210-224); its CUDA path calls cublasSgemm with one
// row (src/cuda_matmul.cpp:216-233).  Here any number of rows runs at once.
//
// One order of summation for every shape.  K is cut into chunks of 256; inside a chunk the
// terms are added in ascending k into one accumulator that starts at zero (fused
// multiply-adds); the chunks' sums are then added in ascending order into a total that
// starts at zero.  Every kernel below produces exactly this sum for every output element,
// so a token's result does not depend, bit for bit, on how many other tokens ran with it
// or on which kernel took the step.
//
// Three shapes of work:
//   many rows (prompts)   tiles of 128 x 128 outputs, 8 x 8 per thread; operands come in
//                         16-byte loads into registers one K step ahead and go through a
//                         double-buffered shared-memory tile;
//   some rows             the same with tiles of 64 x 64, 4 x 4 per thread;
//   few rows (decoding)   tiles of 16 rows x 64 columns.  Such a product is a stream of
//                         weights with almost no arithmetic, and with few columns it has
//                         too few tiles to keep the memory system busy: each block then
//                         takes one chunk of K for its tile and leaves the chunk's sums in
//                         scratch memory, and a second kernel adds the chunks in order.
#include "common.cuh"

namespace mlc {

constexpr int LS_BK = 16;
constexpr int LS_CHUNK = 256;          // a multiple of LS_BK

// Four consecutive elements of a row as floats; `vec` says that 4-element groups of every row are aligned for one load.
template <typename T>
__device__ __forceinline__ float4 load4(const T* __restrict__ base, long long row, int K, int k, bool row_ok, bool vec);

template <>
__device__ __forceinline__ float4 load4<float>(const float* __restrict__ base, long long row, int K, int k, bool row_ok, bool vec) {
    if (!row_ok || k >= K) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float* p = base + row * K + k;
    if (vec && k + 3 < K) return __ldg(reinterpret_cast<const float4*>(p));
    float4 v = make_float4(p[0], 0.0f, 0.0f, 0.0f);
    if (k + 1 < K) v.y = p[1];
    if (k + 2 < K) v.z = p[2];
    if (k + 3 < K) v.w = p[3];
    return v;
}

template <>
__device__ __forceinline__ float4 load4<bf16>(const bf16* __restrict__ base, long long row, int K, int k, bool row_ok, bool vec) {
    if (!row_ok || k >= K) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const bf16* p = base + row * K + k;
    if (vec && k + 3 < K) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    float4 v = make_float4(__bfloat162float(p[0]), 0.0f, 0.0f, 0.0f);
    if (k + 1 < K) v.y = __bfloat162float(p[1]);
    if (k + 2 < K) v.z = __bfloat162float(p[2]);
    if (k + 3 < K) v.w = __bfloat162float(p[3]);
    return v;
}

template <typename T> __device__ __forceinline__ bool rows_vectorizable(const T* base, int K) {
    return (K & 3) == 0 && (reinterpret_cast<uintptr_t>(base) & (4 * sizeof(T) - 1)) == 0;
}

// A tile of BM x BN outputs, TM x TN per thread, over the K range [k_begin, k_end) (whole chunks, but for the matrix's
// end).  `total` starts at zero and gets each chunk's sum in turn.  PARTIAL: the range is one chunk and its sum goes to
// part[chunk][M][N] instead of y.
template <typename TX, typename TW, typename TY, int BM, int BN, int TM, int TN, bool PARTIAL>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
linear_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, float* __restrict__ part,
                   int M, int N, int K) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int XV = (BM * (LS_BK / 4) + THREADS - 1) / THREADS;       // 16-byte loads per thread and K step
    constexpr int WV = (BN * (LS_BK / 4) + THREADS - 1) / THREADS;
    __shared__ __align__(16) float xs[2][LS_BK][BM + 4];
    __shared__ __align__(16) float ws[2][LS_BK][BN + 4];
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_begin = PARTIAL ? blockIdx.z * LS_CHUNK : 0;
    const int k_end = PARTIAL ? min(K, k_begin + LS_CHUNK) : K;
    const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
    const bool x_vec = rows_vectorizable(x, K), w_vec = rows_vectorizable(w, K);

    float total[TM][TN], acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) total[i][j] = acc[i][j] = 0.0f;

    float4 xr[XV], wr[WV];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int v = 0; v < XV; ++v) {
            const int idx = threadIdx.x + v * THREADS, row = idx / (LS_BK / 4), kq = (idx % (LS_BK / 4)) * 4;
            xr[v] = load4<TX>(x, m0 + row, K, k0 + kq, idx < BM * (LS_BK / 4) && m0 + row < M && k0 + kq < k_end, x_vec);
        }
#pragma unroll
        for (int v = 0; v < WV; ++v) {
            const int idx = threadIdx.x + v * THREADS, row = idx / (LS_BK / 4), kq = (idx % (LS_BK / 4)) * 4;
            wr[v] = load4<TW>(w, n0 + row, K, k0 + kq, idx < BN * (LS_BK / 4) && n0 + row < N && k0 + kq < k_end, w_vec);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int v = 0; v < XV; ++v) {
            const int idx = threadIdx.x + v * THREADS, row = idx / (LS_BK / 4), kq = (idx % (LS_BK / 4)) * 4;
            if (idx < BM * (LS_BK / 4)) {
                xs[buf][kq][row] = xr[v].x; xs[buf][kq + 1][row] = xr[v].y; xs[buf][kq + 2][row] = xr[v].z; xs[buf][kq + 3][row] = xr[v].w;
            }
        }
#pragma unroll
        for (int v = 0; v < WV; ++v) {
            const int idx = threadIdx.x + v * THREADS, row = idx / (LS_BK / 4), kq = (idx % (LS_BK / 4)) * 4;
            if (idx < BN * (LS_BK / 4)) {
                ws[buf][kq][row] = wr[v].x; ws[buf][kq + 1][row] = wr[v].y; ws[buf][kq + 2][row] = wr[v].z; ws[buf][kq + 3][row] = wr[v].w;
            }
        }
    };

    fetch(k_begin);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = k_begin; k0 < k_end; k0 += LS_BK) {
        const bool more = k0 + LS_BK < k_end;
        if (more) fetch(k0 + LS_BK);                         // the next step's operands travel while this one is multiplied
        const int steps = min(LS_BK, k_end - k0);            // no term beyond K is ever added
#pragma unroll 4
        for (int kk = 0; kk < steps; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[buf][kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[buf][kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (!PARTIAL && ((k0 + LS_BK) % LS_CHUNK == 0 || !more)) {       // a chunk is complete
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    total[i][j] += acc[i][j];
                    acc[i][j] = 0.0f;
                }
        }
        if (more) {
            stash(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            if (PARTIAL) part[((long long)blockIdx.z * M + m) * N + n] = acc[i][j];
            else y[(long long)m * N + n] = from_float<TY>(total[i][j]);
        }
    }
}

// y = the chunks' sums added in ascending order into a total that starts at zero.
template <typename TY>
__global__ void linear_simt_add_chunks_kernel(const float* __restrict__ part, TY* __restrict__ y, long long MN, int n_chunks) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MN) return;
    float total = 0.0f;
    for (int c = 0; c < n_chunks; ++c) total += part[(long long)c * MN + i];
    y[i] = from_float<TY>(total);
}

template <typename TX, typename TW, typename TY>
static int launch_linear(const void* x, const void* w, void* y, float* scratch, long long scratch_floats, int M, int N, int K,
                         int n_sms, cudaStream_t s) {
    const TX* xp = (const TX*)x;
    const TW* wp = (const TW*)w;
    TY* yp = (TY*)y;
    if (M > 64) {
        dim3 grid((N + 127) / 128, (M + 127) / 128);
        if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
        linear_simt_kernel<TX, TW, TY, 128, 128, 8, 8, false><<<grid, 256, 0, s>>>(xp, wp, yp, nullptr, M, N, K);
    } else if (M > 16) {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        linear_simt_kernel<TX, TW, TY, 64, 64, 4, 4, false><<<grid, 256, 0, s>>>(xp, wp, yp, nullptr, M, N, K);
    } else {
        const int n_chunks = (K + LS_CHUNK - 1) / LS_CHUNK;
        const int tiles = (N + 63) / 64;
        const long long need = (long long)n_chunks * M * N;
        // few tiles: a block per (tile, chunk) and a second kernel that adds the chunks, if the caller gave room for them
        if (tiles < 4 * n_sms && n_chunks > 1 && n_chunks <= 65535 && scratch != nullptr && scratch_floats >= need) {
            dim3 grid(tiles, 1, n_chunks);
            linear_simt_kernel<TX, TW, TY, 16, 64, 2, 4, true><<<grid, 128, 0, s>>>(xp, wp, yp, scratch, M, N, K);
            MLC_LAUNCH_CHECK();
            const long long MN = (long long)M * N;
            linear_simt_add_chunks_kernel<TY><<<(unsigned)((MN + 255) / 256), 256, 0, s>>>(scratch, yp, MN, n_chunks);
        } else {
            dim3 grid(tiles, 1);
            linear_simt_kernel<TX, TW, TY, 16, 64, 2, 4, false><<<grid, 128, 0, s>>>(xp, wp, yp, nullptr, M, N, K);
        }
    }
    MLC_LAUNCH_CHECK();
    return 0;
}

}  // namespace mlc

using namespace mlc;

// Floats of scratch memory a product of these sizes can use (0: none): room for each K chunk's sums when few rows meet
// few columns.  Without it the product still runs, with fewer blocks.
extern "C" long long mlc_linear_simt_scratch_floats(int M, int N, int K, int n_sms) {
    if (M <= 0 || M > 16 || N <= 0 || K <= LS_CHUNK) return 0;
    if ((N + 63) / 64 >= 4 * n_sms) return 0;
    return (long long)((K + LS_CHUNK - 1) / LS_CHUNK) * M * N;
}

// x [M][K] of x_dtype, w [N][K] of w_dtype, y [M][N] of y_dtype; all row-major and dense.  scratch: null, or
// `scratch_floats` floats of device memory (see mlc_linear_simt_scratch_floats).
extern "C" int mlc_linear_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                               int M, int N, int K, float* scratch, long long scratch_floats, int n_sms, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || n_sms < 1) return MLC_ERR_BAD_SIZE;
    if ((x_dtype | w_dtype | y_dtype) & ~1) return MLC_ERR_BAD_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
    switch (code) {
        case 0: return launch_linear<float, float, float>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 1: return launch_linear<float, float, bf16>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 2: return launch_linear<float, bf16, float>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 3: return launch_linear<float, bf16, bf16>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 4: return launch_linear<bf16, float, float>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 5: return launch_linear<bf16, float, bf16>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 6: return launch_linear<bf16, bf16, float>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
        case 7: return launch_linear<bf16, bf16, bf16>(x, w, y, scratch, scratch_floats, M, N, K, n_sms, s);
    }
    return MLC_ERR_BAD_DTYPE;
}

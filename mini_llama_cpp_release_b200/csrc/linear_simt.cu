// y[M][N] = x[M][K] · W[N][K]ᵀ with float32 multiply-adds on the CUDA cores: the linear
// layer of the whole-model 32-bit path, and the fallback for operand types the
// tensor-core kernels do not take.  No tensor-core mode of any precision is involved.
//
// The reference's linear is y = W·x for one row x, W row-major [out, in]
// (src/matmul_optimized.cpp:40-54, 210-224); its CUDA path calls cublasSgemm with one
// row (src/cuda_matmul.cpp:216-233).  Here any number of rows runs at once, and each
// output element is always the same sum in the same order (k ascending in steps of 16,
// one accumulator), whatever M is: a token's result does not depend on its batch.
#include "common.cuh"

namespace mlc {

constexpr int LS_BM = 64, LS_BN = 64, LS_BK = 16, LS_THREADS = 256;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(LS_THREADS)
linear_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y, int M, int N, int K) {
    __shared__ float xs[LS_BK][LS_BM + 4];
    __shared__ float ws[LS_BK][LS_BN + 4];
    const int m0 = blockIdx.y * LS_BM, n0 = blockIdx.x * LS_BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;   // thread's 4x4 patch: rows ty*4.., cols tx*4..
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const int lk = threadIdx.x % LS_BK, lr = threadIdx.x / LS_BK;   // loader: column k, rows lr + 16*i
    for (int k0 = 0; k0 < K; k0 += LS_BK) {
        const int k = k0 + lk;
#pragma unroll
        for (int i = 0; i < LS_BM / 16; ++i) {
            const int r = lr + 16 * i;
            const int m = m0 + r, n = n0 + r;
            xs[lk][r] = (m < M && k < K) ? to_float(x[(long long)m * K + k]) : 0.0f;
            ws[lk][r] = (n < N && k < K) ? to_float(w[(long long)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < LS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(long long)m * N + n] = from_float<TY>(acc[i][j]);
        }
    }
}

template <typename TX, typename TW, typename TY>
static int launch_linear(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t s) {
    dim3 grid((N + LS_BN - 1) / LS_BN, (M + LS_BM - 1) / LS_BM);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    linear_simt_kernel<TX, TW, TY><<<grid, LS_THREADS, 0, s>>>((const TX*)x, (const TW*)w, (TY*)y, M, N, K);
    MLC_LAUNCH_CHECK();
    return 0;
}

}  // namespace mlc

using namespace mlc;

// x [M][K] of x_dtype, w [N][K] of w_dtype, y [M][N] of y_dtype; all row-major and dense.
extern "C" int mlc_linear_simt(const void* x, int x_dtype, const void* w, int w_dtype, void* y, int y_dtype,
                               int M, int N, int K, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return MLC_ERR_BAD_SIZE;
    if ((x_dtype | w_dtype | y_dtype) & ~1) return MLC_ERR_BAD_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
    switch (code) {
        case 0: return launch_linear<float, float, float>(x, w, y, M, N, K, s);
        case 1: return launch_linear<float, float, bf16>(x, w, y, M, N, K, s);
        case 2: return launch_linear<float, bf16, float>(x, w, y, M, N, K, s);
        case 3: return launch_linear<float, bf16, bf16>(x, w, y, M, N, K, s);
        case 4: return launch_linear<bf16, float, float>(x, w, y, M, N, K, s);
        case 5: return launch_linear<bf16, float, bf16>(x, w, y, M, N, K, s);
        case 6: return launch_linear<bf16, bf16, float>(x, w, y, M, N, K, s);
        case 7: return launch_linear<bf16, bf16, bf16>(x, w, y, M, N, K, s);
    }
    return MLC_ERR_BAD_DTYPE;
}

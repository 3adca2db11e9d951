// What the two prompt forms of the tcgen05 product share (tokens as the M operand: gemm_tcgen05_rows.cu with one SM
// per tile, gemm_tcgen05_pair.cu with a pair of SMs): the arguments, and what an epilogue thread does with 32 columns
// of its token's accumulator row.
#pragma once

#include "tcgen05.cuh"

namespace mlc {

enum { R_EPI_STORE = 0, R_EPI_SILU_MUL = 1, R_EPI_QKV = 2, R_EPI_ADD = 3 };

struct RowsArgs {
    void* out;
    int out_dtype;
    int n_out;                 // rows of W = columns of the product; a multiple of 16
    int n_tok;
    int k_blocks;              // ceil(K / 64)
    int m_tiles, n_tiles;
    int n_splits;              // blocks that share out a tile's K range (ADD only); 1: none
    int k_blocks_per_split;
    int* status;
    // QKV epilogue
    const float* bias;         // [n_out] in the stored row order, or null
    const int* positions;      // [tokens]
    const int* tok_seq;        // [tokens]
    const float2* rope;        // [positions][hd/2] cos, sin; or null
    int rope_positions;
    int q_heads, kv_heads, hd;
    PagedKV cache;
};

constexpr int R_BM = 128;
constexpr int R_BK = 64;
constexpr int R_A_BYTES = R_BM * R_BK * 2;

__device__ __forceinline__ unsigned pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&h);
}

// One token's 32 (or, at the matrix's edge, 16) accumulator columns n .. n+31 leave the block.  `second`: the upper 16
// exist too.  STORE: y as float32 or bfloat16; ADD: added into the float32 stream with 16-byte atomic adds (one
// per element and launch unless the K range is shared out over blocks); SILU_MUL: columns alternate gate_j, up_j
// and gate·sigmoid(gate)·up goes to [token][n/2].
template <int EPI>
__device__ __forceinline__ void rows_epilogue_chunk(const RowsArgs& g, const float (&v)[32], int tok, int n, bool second) {
    if (EPI == R_EPI_STORE) {
        if (g.out_dtype == MLC_DTYPE_BF16) {
            uint4* dst = reinterpret_cast<uint4*>((bf16*)g.out + (long long)tok * g.n_out + n);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (u < 2 || second)
                    dst[u] = make_uint4(pack2(v[8 * u], v[8 * u + 1]), pack2(v[8 * u + 2], v[8 * u + 3]),
                                        pack2(v[8 * u + 4], v[8 * u + 5]), pack2(v[8 * u + 6], v[8 * u + 7]));
        } else {
            float4* dst = reinterpret_cast<float4*>((float*)g.out + (long long)tok * g.n_out + n);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (u < 4 || second) dst[u] = make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
        }
    } else if (EPI == R_EPI_ADD) {                    // a reduction that returns nothing: the thread does not wait for the old value
        float4* dst = reinterpret_cast<float4*>((float*)g.out + (long long)tok * g.n_out + n);
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (u < 4 || second) atomicAdd(dst + u, make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]));
    } else {                                          // SILU_MUL: columns alternate gate_j, up_j
        float act[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const float gate = v[2 * u], up = v[2 * u + 1];
            act[u] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
        }
        const long long at = (long long)tok * (g.n_out >> 1) + (n >> 1);
        if (g.out_dtype == MLC_DTYPE_BF16) {
            uint4* dst = reinterpret_cast<uint4*>((bf16*)g.out + at);
            dst[0] = make_uint4(pack2(act[0], act[1]), pack2(act[2], act[3]), pack2(act[4], act[5]), pack2(act[6], act[7]));
            if (second) dst[1] = make_uint4(pack2(act[8], act[9]), pack2(act[10], act[11]), pack2(act[12], act[13]), pack2(act[14], act[15]));
        } else {
            float4* dst = reinterpret_cast<float4*>((float*)g.out + at);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (u < 2 || second) dst[u] = make_float4(act[4 * u], act[4 * u + 1], act[4 * u + 2], act[4 * u + 3]);
        }
    }
}

}  // namespace mlc

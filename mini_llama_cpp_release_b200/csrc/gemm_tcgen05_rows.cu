// y[token][row] = sum_k h[token][k] · W[row][k] for prompts: the same tcgen05 pipeline as gemm_tcgen05.cu
// with the operands the other way round.  The tokens are the M operand (a block owns 128 tokens, UMMA M = 128)
// and BN rows of W are the N operand, so a thread of the epilogue holds one token's run of outputs: partners of
// a rotation pair or of a gate/up pair sit in neighbouring registers instead of neighbouring lanes, and results
// leave in 16-byte stores without a pass through shared memory.  With a handful of tokens the other kernel is
// the one to use (its N can be 16); this one wants at least a tile of 128.
//
//     warp 0    one thread issues the TMA loads of the token tile and the W tile through a ring of stages;
//     warp 1    allocates tensor memory; one thread issues tcgen05.mma and commits;
//     warps 2-9 read the accumulators (warp q its 32 lanes = tokens, the two groups of four warps half of the
//               columns each) and run the epilogue.
// Blocks are persistent (one per SM at most) and keep two accumulators, so one tile's epilogue runs while the
// next tile's products do.
//
// Epilogues (W's rows stored in the same orders as for gemm_tcgen05.cu):
//   STORE     y as float32 or bfloat16, [token][row];
//   SILU_MUL  rows alternate gate_j, up_j: writes gate·sigmoid(gate)·up as [token][row/2] (src/ops.cpp:94-107);
//   QKV       rows of each head alternate dim i, dim i + hd/2: adds the bias, rotates q and k by the token's
//             position (src/ops.cpp:125-141), writes q as [token][head][hd] and k, v into the token's place in
//             the paged cache (src/forward.cpp:553);
//   ADD       adds y into a float32 [token][row] tensor, the residual stream (src/forward.cpp:772, 779), with 16-byte
//             atomic adds: nothing comes back, so a thread does not wait for the stream's old values, and the K
//             range can be shared out over blocks (for products whose tiles alone would leave most SMs idle).
//
// Every wait on an mbarrier is bounded by a clock; a wait that runs out records a code in `status` (21 loader,
// 22 tensor cores, 23 epilogue), the block skips its stores, frees its tensor memory and returns.
#include "gemm_rows_common.cuh"

namespace mlc {

template <int BN> struct RowsShape {
    static constexpr int B_BYTES = BN * R_BK * 2;
    static constexpr int STAGE_BYTES = R_A_BYTES + B_BYTES;
    static constexpr int STAGES_FIT = (227 * 1024 - 256 - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT < 6 ? STAGES_FIT : 6;
    static constexpr int THREADS = 64 + 256;
    static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;    // two accumulators of BN columns; allocations are powers of two
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024 /* alignment slack */;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of a block");
    static_assert(BN % 32 == 0 && BN >= 128 && BN <= 256, "rows of W per tile");
};

template <int BN, int EPI>
__global__ void __launch_bounds__(RowsShape<BN>::THREADS, 1)
gemm_rows_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, RowsArgs g) {
    using S = RowsShape<BN>;
    extern __shared__ unsigned char smem_dyn[];
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    const unsigned a_base = base;
    const unsigned b_base = base + S::STAGES * R_A_BYTES;
    constexpr unsigned bar_off = S::STAGES * S::STAGE_BYTES;
    const unsigned bar_base = base + bar_off;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (8 + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (16 + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (18 + b); };
    const unsigned tmem_slot = bar_base + 8u * 20;
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + bar_off + 8 * 20);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles_total = g.m_tiles * g.n_tiles * g.n_splits;
    // consecutive blocks take the token tiles of one W tile: the W tile is fetched from memory once and then found in L2
    auto tile_m0 = [&](int t) { return (t % g.m_tiles) * R_BM; };
    auto tile_n0 = [&](int t) { return ((t / g.m_tiles) % g.n_tiles) * BN; };
    auto tile_kb0 = [&](int t) { return (t / (g.m_tiles * g.n_tiles)) * g.k_blocks_per_split; };       // first K block of the tile's share
    auto tile_nkb = [&](int t) { return min(g.k_blocks, tile_kb0(t) + g.k_blocks_per_split) - tile_kb0(t); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 256);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((unsigned)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = *tmem_slot_ptr;

    grid_launch_dependents();
    if (warp == 0) {
        // ---------------- TMA producer.  The weights do not depend on the kernels before this one: the first ring of W
        // tiles is requested before the wait for those kernels, the token tiles after it.
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < n_tiles_total && alive; t += gridDim.x) {
                const int m0 = tile_m0(t), n0 = tile_n0(t), kb0 = tile_kb0(t), n_kb = tile_nkb(t);
                int i = 0;
                if (it == 0) {
                    const int early = min(n_kb, S::STAGES);
                    for (; i < early; ++i) {
                        mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                        tma_load_2d(b_base + i * S::B_BYTES, &map_w, (kb0 + i) * R_BK, n0, full_bar(i));
                    }
                    grid_dependency_wait();
                    for (int e = 0; e < early; ++e) tma_load_2d(a_base + e * R_A_BYTES, &map_x, (kb0 + e) * R_BK, m0, full_bar(e));
                    it = early;
                }
                for (; i < n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, g.status, 21)) { alive = false; break; }
                    mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                    tma_load_2d(a_base + s * R_A_BYTES, &map_x, (kb0 + i) * R_BK, m0, full_bar(s));
                    tma_load_2d(b_base + s * S::B_BYTES, &map_w, (kb0 + i) * R_BK, n0, full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: tile j accumulates in buffer j % 2 once the epilogue has emptied it
        if (lane == 0) {
            constexpr unsigned idesc = umma_idesc(BN);
            int it = 0, j = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++j) {
                const int buf = j & 1;
                ok = mbar_wait(acc_empty_bar(buf), (((unsigned)j >> 1) & 1u) ^ 1u, g.status, 22);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
                const int n_kb = tile_nkb(t);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    ok = mbar_wait(full_bar(s), phase, g.status, 22);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const unsigned long long a_desc = umma_desc_sw128(a_base + s * R_A_BYTES);
                    const unsigned long long b_desc = umma_desc_sw128(b_base + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < R_BK / 16; ++k)
                        tcgen05_mma_f16(d_tmem, a_desc + 2ull * k, b_desc + 2ull * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tcgen05_commit(empty_bar(s));
                }
                if (!ok) break;
                tcgen05_commit(acc_full_bar(buf));
            }
        }
    } else {
        // ---------------- epilogue: a thread is one token; the two groups of warps take half of the tile's columns each
        const int q = warp & 3;
        const int eg = (warp - 2) >> 2;
        constexpr int COLS_PER_GROUP = BN / 2;
        grid_dependency_wait();                // positions, page lists and the output may come from earlier kernels
        int j = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++j) {
            const int m0 = tile_m0(t), n0 = tile_n0(t);
            const int buf = j & 1;
            const int tok = m0 + q * 32 + lane;
            const bool tok_ok = tok < g.n_tok;
            int pos = 0;
            long long cache_off = 0;
            if (EPI == R_EPI_QKV && tok_ok) {                        // fetched while the products run
                pos = __ldg(g.positions + tok);
                if (g.kv_heads > 0) cache_off = paged_offset(g.cache, __ldg(g.tok_seq + tok), pos, 0);
            }
            if (EPI != R_EPI_QKV) {
                ok = mbar_wait(acc_full_bar(buf), ((unsigned)j >> 1) & 1u, g.status, 23);
                if (!ok) break;
                tcgen05_fence_after();
            }
            const unsigned t_addr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN + eg * COLS_PER_GROUP);
            const int col_base = n0 + eg * COLS_PER_GROUP;

            if constexpr (EPI == R_EPI_QKV) {
                // 16 columns = 8 rotation pairs of one head (hd is a multiple of 16).  The bias and the token's cos/sin
                // for every chunk are fetched before the accumulator is waited for, so that the products hide the trips
                // to memory; the chunks are unrolled to keep them in registers.
                constexpr int CHUNKS = COLS_PER_GROUP / 16;
                static_assert(CHUNKS <= 4, "the Q/K/V epilogue keeps four chunks of factors in registers: 128-row tiles");
                const int hd = g.hd, half = hd >> 1;
                const float2* rope_row = g.rope == nullptr ? nullptr : g.rope + (long long)min(pos, g.rope_positions - 1) * half;
                float4 cs[CHUNKS][4], bb[CHUNKS][4];
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    const int n = col_base + 16 * c;
                    const int head = n / hd, i0 = (n % hd) >> 1;
                    const bool rotate = n < g.n_out && head < g.q_heads + g.kv_heads && rope_row != nullptr && tok_ok;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        cs[c][u] = rotate ? __ldg(reinterpret_cast<const float4*>(rope_row + i0) + u) : make_float4(1.0f, 0.0f, 1.0f, 0.0f);
                        bb[c][u] = (g.bias != nullptr && n < g.n_out) ? __ldg(reinterpret_cast<const float4*>(g.bias + n) + u)
                                                                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                }
                ok = mbar_wait(acc_full_bar(buf), ((unsigned)j >> 1) & 1u, g.status, 23);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    const int n = col_base + 16 * c;
                    if (n < g.n_out) {                                // the same for the whole warp
                        float v[16];
                        tmem_load16(t_addr + (unsigned)(16 * c), v);
                        const int head = n / hd, i0 = (n % hd) >> 1;
                        const bool is_q = head < g.q_heads;
                        const bool is_k = !is_q && head < g.q_heads + g.kv_heads;
                        float lo[8], hi[8];                           // dims i0 .. i0+7 and i0 + hd/2 .. of the head
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float4 f = cs[c][u], b = bb[c][u];
                            const float x0 = v[4 * u] + b.x, x1 = v[4 * u + 1] + b.y, y0 = v[4 * u + 2] + b.z, y1 = v[4 * u + 3] + b.w;
                            lo[2 * u] = x0 * f.x - x1 * f.y;          // (cos, sin) = (1, 0) where nothing is rotated
                            hi[2 * u] = x0 * f.y + x1 * f.x;
                            lo[2 * u + 1] = y0 * f.z - y1 * f.w;
                            hi[2 * u + 1] = y0 * f.w + y1 * f.z;
                        }
                        if (tok_ok) {
                            bf16* dst;
                            if (is_q) dst = (bf16*)g.out + ((long long)tok * g.q_heads + head) * hd;
                            else {
                                const int kvh = is_k ? head - g.q_heads : head - g.q_heads - g.kv_heads;
                                dst = (bf16*)(is_k ? g.cache.k_pool : g.cache.v_pool) + cache_off + (long long)kvh * g.cache.page_size * hd;
                            }
                            *reinterpret_cast<uint4*>(dst + i0) = make_uint4(pack2(lo[0], lo[1]), pack2(lo[2], lo[3]), pack2(lo[4], lo[5]), pack2(lo[6], lo[7]));
                            *reinterpret_cast<uint4*>(dst + half + i0) = make_uint4(pack2(hi[0], hi[1]), pack2(hi[2], hi[3]), pack2(hi[4], hi[5]), pack2(hi[6], hi[7]));
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < COLS_PER_GROUP; c0 += 32) {
                    const int n = col_base + c0;
                    if (n >= g.n_out) break;
                    float v[32];
                    tmem_load32(t_addr + (unsigned)c0, v);
                    // n_out and the group's share of the tile are multiples of 16: the chunk has 16 or 32 columns
                    const bool second = n + 16 < g.n_out && c0 + 32 <= COLS_PER_GROUP;
                    if (!tok_ok) continue;
                    rows_epilogue_chunk<EPI>(g, v, tok, n, second);
                }
            }
            // the accumulator has been read: the tensor cores may fill it again
            tcgen05_fence_before();
            mbar_arrive(acc_empty_bar(buf));
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS) : "memory");
    }
}

// A row-major bfloat16 matrix [rows][cols] read in boxes of box_rows x 64 columns.
static int rows_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    return cached_map_2d(map, ptr, rows, cols, R_BK, box_rows);
}

template <int BN, int EPI>
static int launch_rows(const CUtensorMap& mx, const CUtensorMap& mw, const RowsArgs& g, int n_sms, cudaStream_t s) {
    using S = RowsShape<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_rows_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long tiles = (long long)g.m_tiles * g.n_tiles * g.n_splits;
    const unsigned blocks = (unsigned)(tiles < n_sms ? tiles : n_sms);
    cudaError_t e = launch_pdl(gemm_rows_kernel<BN, EPI>, dim3(blocks), dim3(S::THREADS), (size_t)S::SMEM_BYTES, s, mx, mw, g);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int EPI>
static int dispatch_rows(int bn, const CUtensorMap& mx, const CUtensorMap& mw, const RowsArgs& g, int n_sms, cudaStream_t s) {
    if (bn == 128) return launch_rows<128, EPI>(mx, mw, g, n_sms, s);
    if (bn == 160) return launch_rows<160, EPI>(mx, mw, g, n_sms, s);
    if (bn == 192) return launch_rows<192, EPI>(mx, mw, g, n_sms, s);
    if (bn == 224) return launch_rows<224, EPI>(mx, mw, g, n_sms, s);
    if (bn == 256) return launch_rows<256, EPI>(mx, mw, g, n_sms, s);
    return MLC_ERR_BAD_SIZE;
}

}  // namespace mlc

using namespace mlc;

// x: bfloat16 [n_tok][K]; w: bfloat16 [n_out][K]; K a multiple of 8, n_out a multiple of 16, everything 16-byte
// aligned.  block_rows: 128, 160, 192, 224 or 256 rows of W per tile.  epilogue 0: out [n_tok][n_out] float32 or bfloat16; 1: out
// [n_tok][n_out/2]; 2: out = q [n_tok][q_heads*hd] bfloat16, k and v go to the bfloat16 cache (hd a multiple of 16; block_rows 128);
// 3: adds into out, float32 [n_tok][n_out]; n_splits > 1 (this epilogue only) shares the K range out over that many
// blocks per tile, which then add atomically.  status: one int on the device, 0 before the call; a bounded wait that
// ran out leaves 21 (loader), 22 (tensor cores) or 23 (epilogue) there.  n_sms: blocks to launch at most.
extern "C" int mlc_gemm_tcgen05_rows(const void* x, const void* w, void* out, int out_dtype, int n_tok, int n_out, int K,
                                     int block_rows, int n_splits, int epilogue, int* status, int n_sms, const float* bias,
                                     const int* positions, const int* tok_seq, const void* rope_table, int rope_positions,
                                     int q_heads, int kv_heads, int hd, void* k_pool, void* v_pool, const int* page_table,
                                     long long entry_offset, int pages_per_seq, int page_size, void* stream) {
    if (n_tok <= 0 || n_out <= 0) return 0;
    if (K <= 0 || (K & 7) || (n_out & 15) || (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15)) return MLC_ERR_BAD_SIZE;
    if (out_dtype != MLC_DTYPE_F32 && out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    if (status == nullptr || n_sms < 1) return MLC_ERR_BAD_SIZE;
    if (epilogue == R_EPI_ADD && out_dtype != MLC_DTYPE_F32) return MLC_ERR_BAD_DTYPE;
    if (n_splits < 1 || (n_splits > 1 && epilogue != R_EPI_ADD)) return MLC_ERR_BAD_SIZE;
    RowsArgs g{};
    g.out = out;
    g.out_dtype = out_dtype;
    g.n_out = n_out;
    g.n_tok = n_tok;
    g.k_blocks = (K + R_BK - 1) / R_BK;
    g.m_tiles = (n_tok + R_BM - 1) / R_BM;
    g.n_tiles = (n_out + block_rows - 1) / block_rows;
    g.n_splits = n_splits;
    g.k_blocks_per_split = (g.k_blocks + n_splits - 1) / n_splits;
    if ((long long)(n_splits - 1) * g.k_blocks_per_split >= g.k_blocks) return MLC_ERR_BAD_SIZE;   // an empty split
    g.status = status;
    if (epilogue == R_EPI_QKV) {
        if (out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
        if (hd <= 0 || (hd & 15) || n_out != (q_heads + 2 * kv_heads) * hd || positions == nullptr) return MLC_ERR_BAD_SIZE;
        if (kv_heads > 0 && (tok_seq == nullptr || k_pool == nullptr || v_pool == nullptr || page_table == nullptr)) return MLC_ERR_BAD_SIZE;
        if ((((uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)bias | (uintptr_t)rope_table) & 15) || (entry_offset & 7)) return MLC_ERR_BAD_SIZE;
        g.bias = bias;
        g.positions = positions;
        g.tok_seq = tok_seq;
        g.rope = (const float2*)rope_table;
        g.rope_positions = rope_positions;
        g.q_heads = q_heads;
        g.kv_heads = kv_heads;
        g.hd = hd;
        g.cache = PagedKV{k_pool, v_pool, page_table, entry_offset, pages_per_seq, page_size, kv_heads, hd};
    }
    CUtensorMap mx, mw;
    int rc = rows_map(&mx, x, n_tok, K, R_BM);
    if (rc) return rc;
    rc = rows_map(&mw, w, n_out, K, block_rows);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == R_EPI_STORE) return dispatch_rows<R_EPI_STORE>(block_rows, mx, mw, g, n_sms, s);
    if (epilogue == R_EPI_SILU_MUL) return dispatch_rows<R_EPI_SILU_MUL>(block_rows, mx, mw, g, n_sms, s);
    if (epilogue == R_EPI_QKV) return block_rows == 128 ? launch_rows<128, R_EPI_QKV>(mx, mw, g, n_sms, s) : MLC_ERR_BAD_SIZE;
    if (epilogue == R_EPI_ADD) return dispatch_rows<R_EPI_ADD>(block_rows, mx, mw, g, n_sms, s);
    return MLC_ERR_UNSUPPORTED;
}

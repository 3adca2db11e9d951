// y[token][row] = sum_k h[token][k] · W[row][k] for prompts, with a pair of SMs on every tile.
//
// The one-SM form of this product (gemm_tcgen05_rows.cu) is bound by what an SM can draw from L2: a tile of 128
// tokens x 224 rows of W needs 44 KB per K step for 470 tensor-core clocks.  Here two blocks of a thread-block
// cluster share a tile of 256 tokens x BN rows of W (tcgen05.mma.cta_group::2, UMMA M = 256): each block loads its
// own 128 tokens and its own half of the W rows, the tensor cores of both SMs read both halves, and each block ends
// up with its 128 tokens x BN columns in its own tensor memory.  Per product a block draws a third less.
//
//     warp 0    one thread issues the TMA loads of the block's token tile and its half of the W tile;
//     warp 1    allocates tensor memory (both blocks, together).  In the pair's first block one thread issues
//               tcgen05.mma for the pair and commits to barriers of both blocks; in the second block one thread tells
//               the first when a stage of its shared memory has landed (a remote arrive on a barrier of the first);
//     warps 2-9 read the block's accumulators and run the epilogue, as in the one-SM form.
// Loads carry no cluster qualifier of any kind: every block fetches what it needs itself.
//
// Epilogues: STORE, SILU_MUL, ADD (gemm_rows_common.cuh); ADD may share the K range out over pairs.  The Q/K/V
// epilogue stays with the one-SM form.  Every wait is bounded by a clock; a wait that runs out records a code in
// `status` (41 loader, 42 tensor cores or relay, 43 epilogue), the block skips its stores and leaves.
#include "gemm_rows_common.cuh"

namespace mlc {

template <int BN> struct PairShape {
    static constexpr int B_BYTES = (BN / 2) * R_BK * 2;              // this block's half of the W tile
    static constexpr int STAGE_BYTES = R_A_BYTES + B_BYTES;
    static constexpr int STAGES_FIT = (227 * 1024 - 512 - 1024) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT < 7 ? STAGES_FIT : 7;
    static constexpr int THREADS = 64 + 256;
    static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;    // two accumulators of BN columns
    static constexpr int BAR_BYTES = 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024 /* alignment slack */;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of a block");
    static_assert(BN % 32 == 0 && BN >= 128 && BN <= 256, "rows of W per tile");
    static_assert(STAGES >= 3 && STAGES <= 8, "stage ring");
};

// A remote arrival (mbar_arrive_remote) without ordering of this thread's own earlier writes (it has none to publish): what the arrival reports was
// written by the TMA unit and was complete before the local barrier said so.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                                     unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the products issued so far are done, on the barrier at this address in both blocks of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(unsigned bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
// Instruction descriptor of the pair's product: bfloat16 x bfloat16 -> float32, both operands K-major, M = 256, N = n.
__host__ __device__ constexpr unsigned umma_idesc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
}

template <int BN, int EPI>
__global__ void __launch_bounds__(PairShape<BN>::THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, RowsArgs g) {
    using S = PairShape<BN>;
    extern __shared__ unsigned char smem_dyn[];
    const unsigned rank = cluster_rank();                  // 0: the block that issues the pair's products
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    const unsigned a_base = base;
    const unsigned b_base = base + S::STAGES * R_A_BYTES;
    constexpr unsigned bar_off = S::STAGES * S::STAGE_BYTES;
    const unsigned bar_base = base + bar_off;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };                // this block's stage has landed
    auto empty_bar = [&](int s) { return bar_base + 8u * (8 + s); };         // the pair's products have read the stage (both blocks)
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (24 + b); };     // the tile's products are done (both blocks)
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (26 + b); };    // first block only: both blocks have read the accumulator
    const unsigned tmem_slot = bar_base + 8u * 28;
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + bar_off + 8 * 28);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_tiles_total = g.m_tiles * g.n_tiles * g.n_splits;           // m_tiles counts tiles of 256 tokens
    auto tile_m0 = [&](int t) { return (t % g.m_tiles) * 2 * R_BM + (int)rank * R_BM; };             // this block's 128 tokens
    auto tile_n0 = [&](int t) { return ((t / g.m_tiles) % g.n_tiles) * BN; };
    auto tile_kb0 = [&](int t) { return (t / (g.m_tiles * g.n_tiles)) * g.k_blocks_per_split; };
    auto tile_nkb = [&](int t) { return min(g.k_blocks, tile_kb0(t) + g.k_blocks_per_split) - tile_kb0(t); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(full_bar(s), rank == 0 ? 2 : 1);     // first block: its own loads, and the second block's word that its stage has landed
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), 2);                // one arrival from each block's epilogue
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // both blocks' barriers exist before either block's loads, commits or remote arrivals can reach them
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((unsigned)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = *tmem_slot_ptr;

    grid_launch_dependents();
    if (warp == 0) {
        // ---------------- TMA producer of this block: its 128 tokens and its BN/2 rows of W.  The first ring of W tiles
        // is requested before the wait for the kernels before this one, the token tiles after it.
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int t = pair; t < n_tiles_total && alive; t += n_pairs) {
                const int m0 = tile_m0(t), w0 = tile_n0(t) + (int)rank * (BN / 2), kb0 = tile_kb0(t), n_kb = tile_nkb(t);
                int i = 0;
                if (it == 0) {
                    const int early = min(n_kb, S::STAGES);
                    for (; i < early; ++i) {
                        mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                        tma_load_2d(b_base + i * S::B_BYTES, &map_w, (kb0 + i) * R_BK, w0, full_bar(i));
                    }
                    grid_dependency_wait();
                    for (int e = 0; e < early; ++e) tma_load_2d(a_base + e * R_A_BYTES, &map_x, (kb0 + e) * R_BK, m0, full_bar(e));
                    it = early;
                }
                for (; i < n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, g.status, 41)) { alive = false; break; }
                    mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                    tma_load_2d(a_base + s * R_A_BYTES, &map_x, (kb0 + i) * R_BK, m0, full_bar(s));
                    tma_load_2d(b_base + s * S::B_BYTES, &map_w, (kb0 + i) * R_BK, w0, full_bar(s));
                }
            }
        }
    } else if (warp == 1 && rank == 1) {
        // ---------------- second block: every stage that has landed here is reported to the first block, whose
        // products read it: a second arrival on the first block's barrier of that stage
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            unsigned remote[S::STAGES];
#pragma unroll
            for (int s = 0; s < S::STAGES; ++s) remote[s] = cluster_map(full_bar(s), 0);
            for (int t = pair; t < n_tiles_total && ok; t += n_pairs) {
                const int n_kb = tile_nkb(t);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    ok = mbar_wait_polling(full_bar(s), (it / S::STAGES) & 1, g.status, 42);    // on the first block's critical path
                    if (!ok) break;
                    unsigned addr = remote[0];
#pragma unroll
                    for (int u = 1; u < S::STAGES; ++u) addr = (s == u) ? remote[u] : addr;
                    mbar_arrive_remote_relaxed(addr);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- first block: the pair's products.  Tile j accumulates in buffer j % 2 of both blocks once
        // both epilogues have emptied it.
        if (lane == 0) {
            constexpr unsigned idesc = umma_idesc_pair(BN);
            int it = 0, j = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles_total && ok; t += n_pairs, ++j) {
                const int buf = j & 1;
                ok = mbar_wait_cluster(acc_empty_bar(buf), (((unsigned)j >> 1) & 1u) ^ 1u, g.status, 42);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
                const int n_kb = tile_nkb(t);
                for (int i = 0; i < n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    ok = mbar_wait_polling(full_bar(s), phase, g.status, 42);        // both blocks' stages have landed
                    if (!ok) break;
                    tcgen05_fence_after();
                    const unsigned long long a_desc = umma_desc_sw128(a_base + s * R_A_BYTES);
                    const unsigned long long b_desc = umma_desc_sw128(b_base + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < R_BK / 16; ++k)
                        tcgen05_mma_f16_pair(d_tmem, a_desc + 2ull * k, b_desc + 2ull * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tcgen05_commit_pair(empty_bar(s));               // both blocks may refill the stage once these products have read it
                }
                if (!ok) break;
                tcgen05_commit_pair(acc_full_bar(buf));
            }
        }
    } else {
        // ---------------- epilogue: a thread is one of this block's tokens; the two groups of warps take half of the
        // tile's columns each
        const int q = warp & 3;
        const int eg = (warp - 2) >> 2;
        constexpr int COLS_PER_GROUP = BN / 2;
        grid_dependency_wait();                // the output may come from earlier kernels
        int j = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles_total && ok; t += n_pairs, ++j) {
            const int m0 = tile_m0(t), n0 = tile_n0(t);
            const int buf = j & 1;
            const int tok = m0 + q * 32 + lane;
            const bool tok_ok = tok < g.n_tok;
            ok = mbar_wait(acc_full_bar(buf), ((unsigned)j >> 1) & 1u, g.status, 43);
            if (!ok) break;
            tcgen05_fence_after();
            const unsigned t_addr = tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN + eg * COLS_PER_GROUP);
            const int col_base = n0 + eg * COLS_PER_GROUP;
#pragma unroll 1
            for (int c0 = 0; c0 < COLS_PER_GROUP; c0 += 32) {
                const int n = col_base + c0;
                if (n >= g.n_out) break;
                float v[32];
                tmem_load32(t_addr + (unsigned)c0, v);
                const bool second = n + 16 < g.n_out && c0 + 32 <= COLS_PER_GROUP;
                if (!tok_ok) continue;
                rows_epilogue_chunk<EPI>(g, v, tok, n, second);
            }
            // the accumulator has been read here: once the other block's has been too, the tensor cores may fill it again
            tcgen05_fence_before();
            asm volatile("bar.sync 1, 256;" ::: "memory");                   // the epilogue warps only
            if (threadIdx.x == 64) {
                if (rank == 0) mbar_arrive(acc_empty_bar(buf));
                else mbar_arrive_remote(cluster_map(acc_empty_bar(buf), 0));
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    // neither block leaves (or gives its tensor memory back) while the other may still read its shared memory or
    // signal its barriers
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS) : "memory");
    }
}

template <int BN, int EPI>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const RowsArgs& g, int n_sms, cudaStream_t s) {
    using S = PairShape<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long tiles = (long long)g.m_tiles * g.n_tiles * g.n_splits;
    const long long pairs = tiles < n_sms / 2 ? tiles : n_sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(S::THREADS);
    cfg.dynamicSmemBytes = S::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;       // blocks 2p and 2p + 1 are a pair
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, EPI>, mx, mw, g);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int EPI>
static int dispatch_pair(int bn, const CUtensorMap& mx, const CUtensorMap& mw, const RowsArgs& g, int n_sms, cudaStream_t s) {
    if (bn == 128) return launch_pair<128, EPI>(mx, mw, g, n_sms, s);
    if (bn == 160) return launch_pair<160, EPI>(mx, mw, g, n_sms, s);
    if (bn == 192) return launch_pair<192, EPI>(mx, mw, g, n_sms, s);
    if (bn == 224) return launch_pair<224, EPI>(mx, mw, g, n_sms, s);
    if (bn == 256) return launch_pair<256, EPI>(mx, mw, g, n_sms, s);
    return MLC_ERR_BAD_SIZE;
}

}  // namespace mlc

using namespace mlc;

// x: bfloat16 [n_tok][K]; w: bfloat16 [n_out][K]; K a multiple of 8, n_out a multiple of 16, everything 16-byte
// aligned.  block_rows: 128, 160, 192, 224 or 256 rows of W per tile of 256 tokens.  epilogue 0: out [n_tok][n_out]
// float32 or bfloat16; 1: out [n_tok][n_out/2]; 3: adds into out, float32 [n_tok][n_out], n_splits > 1 shares the K range
// out over that many pairs per tile, which then add atomically.  status: one int on the device, 0 before the call; a
// bounded wait that ran out leaves 41, 42 or 43 there.  n_sms: blocks to launch at most (an even number is used).
extern "C" int mlc_gemm_tcgen05_pair(const void* x, const void* w, void* out, int out_dtype, int n_tok, int n_out, int K,
                                     int block_rows, int n_splits, int epilogue, int* status, int n_sms, void* stream) {
    if (n_tok <= 0 || n_out <= 0) return 0;
    if (K <= 0 || (K & 7) || (n_out & 15) || (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15)) return MLC_ERR_BAD_SIZE;
    if (out_dtype != MLC_DTYPE_F32 && out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    if (status == nullptr || n_sms < 2) return MLC_ERR_BAD_SIZE;
    if (epilogue == R_EPI_ADD && out_dtype != MLC_DTYPE_F32) return MLC_ERR_BAD_DTYPE;
    if (n_splits < 1 || (n_splits > 1 && epilogue != R_EPI_ADD)) return MLC_ERR_BAD_SIZE;
    RowsArgs g{};
    g.out = out;
    g.out_dtype = out_dtype;
    g.n_out = n_out;
    g.n_tok = n_tok;
    g.k_blocks = (K + R_BK - 1) / R_BK;
    g.m_tiles = (n_tok + 2 * R_BM - 1) / (2 * R_BM);
    g.n_tiles = (n_out + block_rows - 1) / block_rows;
    g.n_splits = n_splits;
    g.k_blocks_per_split = (g.k_blocks + n_splits - 1) / n_splits;
    if ((long long)(n_splits - 1) * g.k_blocks_per_split >= g.k_blocks) return MLC_ERR_BAD_SIZE;   // an empty split
    g.status = status;
    CUtensorMap mx, mw;
    int rc = cached_map_2d(&mx, x, n_tok, K, R_BK, R_BM);
    if (rc) return rc;
    rc = cached_map_2d(&mw, w, n_out, K, R_BK, block_rows / 2);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == R_EPI_STORE) return dispatch_pair<R_EPI_STORE>(block_rows, mx, mw, g, n_sms, s);
    if (epilogue == R_EPI_SILU_MUL) return dispatch_pair<R_EPI_SILU_MUL>(block_rows, mx, mw, g, n_sms, s);
    if (epilogue == R_EPI_ADD) return dispatch_pair<R_EPI_ADD>(block_rows, mx, mw, g, n_sms, s);
    return MLC_ERR_UNSUPPORTED;
}

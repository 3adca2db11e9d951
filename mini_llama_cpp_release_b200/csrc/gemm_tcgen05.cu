// y[token][row] = sum_k W[row][k] · h[token][k] on the fifth-generation tensor cores:
// bfloat16 operands staged in shared memory by TMA, float32 accumulators in tensor memory,
// epilogues that finish the layer's arithmetic before anything is written.
//
// The weight matrix is the M operand: a block owns 128 rows of W (UMMA M = 128) and BN
// tokens (UMMA N = 16 ... 256), so the same kernel streams weights once for a handful of
// decoded tokens and tiles a prompt of thousands.  K runs in steps of 64 elements (one
// 128-byte swizzle span per row) through a ring of shared-memory stages:
//     warp 0   one thread issues the TMA loads of the W tile and the activation tile;
//     warp 1   allocates tensor memory, one thread issues tcgen05.mma and commits; for tiles of up to 32 tokens a
//              thread of each of warps 2-4 issues too: the four take K steps in turn into accumulators of their own (an issue
//              costs its thread about sixty clocks however small the product, and one thread's rate would bound the
//              K loop);
//     the next four warps (eight for tiles of 64 tokens and more) read the accumulators with tcgen05.ld (each warp its
//              32 lanes), add the issuers' accumulators and run the epilogue.
// A K range can be split over blocks (blockIdx.z); partial sums then go to separate slices of
// the output and the consumer adds them.
//
// Epilogues (rows of W may be stored in an order that puts partners on neighbouring lanes):
//   STORE     y as float32 or bfloat16, [token][row];
//   SILU_MUL  rows alternate gate_j, up_j: writes gate·sigmoid(gate)·up as [token][row/2]
//             (src/ops.cpp:94-107);
//   QKV       rows of each head alternate dim i, dim i + hd/2: adds the bias, rotates q and k
//             by the token's position (src/ops.cpp:125-141), writes q as [token][head][hd] and
//             k, v into the token's place in the paged cache (src/forward.cpp:553).
//
//   ADD       adds y into a float32 [token][row] tensor (the residual stream) with atomic adds,
//             so that any number of K splits can feed it (src/forward.cpp:772, 779).
// The Q/K/V product of a few tokens has few tiles (nine at 1,152 rows), and a block alone draws its 128 rows of W
// at one SM's pace.  Its K range can therefore be shared out over a thread-block cluster of 2 or 4 blocks, one tile
// and one K range per block: every block fills an accumulator with its part, each of its four epilogue warps
// stores its 32 rows' partial sums into the shared memory of the block that owns those rows (rank = rows' quarter
// · blocks / 4) and arrives on that block's barrier; the owner's warp adds the parts up in a fixed order and
// runs the epilogue (bias, rotation, cache write) on its rows.
// Blocks are persistent: at most one per SM, each walks output tiles t, t + blocks, ...; a block keeps two
// accumulators in tensor memory, so the epilogue of one tile runs while the tensor cores fill the next.
// Tiles of 64 tokens and more have two groups of four epilogue warps that share out the tokens.
//
// Every wait on an mbarrier is bounded by a clock; a wait that runs out records a code in
// `status`, the block skips its stores, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace mlc {

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_A_BYTES = G_BM * G_BK * 2;                 // 16 KiB per stage

enum { EPI_STORE = 0, EPI_SILU_MUL = 1, EPI_QKV = 2, EPI_ADD = 3,
       EPI_QKV_CLUSTER = 4 };      // QKV whose tiles' K range is shared out over a cluster: a kernel of its own, so that the
                                   // plain form keeps its registers (166 against 157 with the exchange compiled in, and a
                                   // decode step of the 0.5B sizes 0.02 ms longer)
__host__ __device__ constexpr bool qkv_epilogue(int epi) { return epi == EPI_QKV || epi == EPI_QKV_CLUSTER; }

struct GemmArgs {
    void* out;                 // STORE / SILU_MUL: [splits][tokens][n_out or n_out/2]; QKV: q [tokens][q_heads*hd]
    int out_dtype;
    int n_out;                 // rows of W
    int n_tok;
    int k_blocks;              // ceil(K / 64)
    int k_blocks_per_split;
    long long split_stride;    // elements between the output slices of two splits
    int* status;
    int m_tiles, n_tiles, n_splits;   // the grid of output tiles the persistent blocks walk
    int cluster_split;         // QKV epilogue: the n_splits blocks of a tile are a cluster and merge their parts (one tile per block)
    unsigned long long* timing;  // [blocks][8] nanosecond stamps of a block's phases, or null; read only in builds with -DMLC_PHASE_STAMPS
    // QKV epilogue
    const float* bias;         // [n_out] in the stored row order, or null
    const int* positions;      // [tokens]
    const int* tok_seq;        // [tokens]
    const float2* rope;        // [positions][hd/2] cos, sin; or null
    int rope_positions;
    int q_heads, kv_heads, hd;
    PagedKV cache;
};

template <int BN, int EPI> struct GemmShape {
    static constexpr int B_BYTES = BN * G_BK * 2;
    static constexpr int STAGE_BYTES = G_A_BYTES + B_BYTES;
    static constexpr int EPI_GROUPS = (BN >= 64) ? 2 : 1;            // epilogue warps: four per group, groups share out the tokens
    // Threads that issue tcgen05.mma.  An issue costs the thread some sixty clocks and a wait on a stage's barrier twice
    // that, whatever the size of the product: with few tokens (tiny products) one thread's issue rate, not the tensor
    // cores, bounds the K loop.  Four threads then take K steps in turn, each into accumulators of its own; the epilogue
    // adds them.
    static constexpr int ISSUERS = (BN <= 32) ? 4 : 1;
    static constexpr int THREADS = 32 + 32 * ISSUERS + 128 * EPI_GROUPS;
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;                // tensor-memory columns of one accumulator
    static constexpr int TMEM_COLS = 2 * ISSUERS * ACC_COLS;          // per issuer two accumulators: one is read out while the other fills
    static constexpr int META_BYTES = BN * 16;                        // per token: position, cache offset (QKV epilogue)
    // SILU_MUL: [8 or 4 warps][tokens][16 outputs] bfloat16; QKV: [8 or 4 warps][2 buffers][16 tokens][32 outputs] bfloat16
    static constexpr int STAGING_BYTES = (EPI == EPI_SILU_MUL) ? 128 * BN : (qkv_epilogue(EPI) ? EPI_GROUPS * 4 * 2048 : 0);
    // QKV: cos and sin of each warp's 16 rotation pairs for the tokens of its group, [warps][tokens][16] float2
    static constexpr int ROPE_BYTES = (qkv_epilogue(EPI) && BN <= 128) ? 4 * BN * 128 : 0;
    // QKV with 16-token tiles: what the blocks of a cluster send this one, [source block][warp of this block's rows][lane][16 tokens]
    // float32: 2 blocks x 2 warps or 4 blocks x 1 warp, 8 KiB.  It lies over the staging tiles: a warp that owns rows
    // reads the parts sent to it (slots source x warps + its number among the owner's warps) before it stages
    // anything, its staging tile (2 KiB at its quarter's number) is one of its own slots, and warps that own no rows
    // stage nothing.
    static constexpr int RECV_BYTES = (EPI == EPI_QKV_CLUSTER && BN == 16) ? 4 * 32 * 16 * 4 : 0;
    static_assert(RECV_BYTES <= STAGING_BYTES, "the received parts lie over the staging tiles");
    static constexpr int BAR_BYTES = 512;                           // up to 16 stages: full 0-15, empty 16-31, accumulators 32-35, slot 36, parts received 37
    static constexpr int FIXED_BYTES = STAGING_BYTES + ROPE_BYTES + BAR_BYTES + META_BYTES + 1024 /* alignment slack */;
    static constexpr int STAGES_FIT = (227 * 1024 - FIXED_BYTES) / STAGE_BYTES;
    // Few tokens: a deep ring, so that as much of a tile's weights as fits is requested before the wait for the kernel
    // before (they depend on nothing) and arrives while it finishes.  Measured on whole decode steps: 8 stages do as well
    // as 12 (0.72 ms at 896 columns, 2.96 against 2.98 ms at 3,584), 4 are a fifth slower (0.85 and 4.06 ms).
    static constexpr int STAGES_WANTED = (BN <= 32) ? 12 : (BN <= 64 ? 8 : (BN <= 128 ? 6 : (EPI == EPI_SILU_MUL ? 3 : 4)));
    // a multiple of ISSUERS: stage s then always belongs to issuer s % ISSUERS, who sees its barrier's phases in order
    static constexpr int STAGES = (STAGES_FIT < STAGES_WANTED ? STAGES_FIT : STAGES_WANTED) / ISSUERS * ISSUERS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + FIXED_BYTES;
    static_assert(STAGES >= 2 && STAGES <= 16, "stage ring");
};

template <typename T> __device__ __forceinline__ void store_out(void* base, long long idx, float v) {
    ((T*)base)[idx] = from_float<T>(v);
}

// One output tile: 128 rows of W x BN tokens x one K range.
struct TileCoord {
    int m0, n0, split, kb_begin, n_kb;
};
// CLUSTERS: the kernel variant can run as clusters that share a tile's K range (the others are spared the test and
// the divisions: every role of every block works a tile's place out before it can ask for anything).
template <bool CLUSTERS>
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& g, int t, int bn) {
    TileCoord c;
    int m_tile, r;
    if (CLUSTERS && g.cluster_split) {         // the blocks of a cluster are neighbours: the splits of a tile run fastest
        const int tile = t / g.n_splits;
        m_tile = tile % g.m_tiles;
        r = (tile / g.m_tiles) + g.n_tiles * (t % g.n_splits);
    } else {
        m_tile = t % g.m_tiles;
        r = t / g.m_tiles;
    }
    c.m0 = m_tile * G_BM;
    c.n0 = (r % g.n_tiles) * bn;
    c.split = r / g.n_tiles;
    c.kb_begin = c.split * g.k_blocks_per_split;
    c.n_kb = min(g.k_blocks, c.kb_begin + g.k_blocks_per_split) - c.kb_begin;
    return c;
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GemmShape<BN, EPI>::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmArgs g) {
    using S = GemmShape<BN, EPI>;
    constexpr int EG = S::EPI_GROUPS;
    extern __shared__ unsigned char smem_dyn[];
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;          // tiles want 1024-byte alignment
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    const unsigned a_base = base;
    const unsigned b_base = base + S::STAGES * G_A_BYTES;
    constexpr unsigned staging_off = S::STAGES * S::STAGE_BYTES;
    constexpr unsigned rope_off = staging_off + S::STAGING_BYTES;
    constexpr unsigned recv_off = staging_off;
    constexpr unsigned bar_off = rope_off + S::ROPE_BYTES;
    const unsigned bar_base = base + bar_off;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (16 + s); };
    auto acc_full_bar = [&](int b) { return bar_base + 8u * (32 + b); };
    auto acc_empty_bar = [&](int b) { return bar_base + 8u * (34 + b); };
    const unsigned recv_bar = bar_base + 8u * 37;
    const bool clustered = S::RECV_BYTES > 0 && g.cluster_split;
    const unsigned tmem_slot = bar_base + 8u * 36;
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + bar_off + 8 * 36);
    int* tok_pos = reinterpret_cast<int*>(smem_generic + bar_off + S::BAR_BYTES);                         // [BN]
    long long* tok_off = reinterpret_cast<long long*>(tok_pos + BN);                                      // [BN]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles_total = g.m_tiles * g.n_tiles * g.n_splits;
    unsigned long long* const stamps = MLC_STAMPS_OR_NULL(g.timing == nullptr ? nullptr : g.timing + 8ull * blockIdx.x);
    if (stamps != nullptr && threadIdx.x == 0) stamps[0] = global_ns();                 // block start

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), S::ISSUERS);
            mbar_init(acc_empty_bar(b), 128 * EG);
        }
        if (S::RECV_BYTES > 0) mbar_init(recv_bar, 128);             // every lane of the four warps that hold this block's rows, in whichever block
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
    if (stamps != nullptr && threadIdx.x == 0) stamps[1] = global_ns();                 // barriers and tensor memory ready

    grid_launch_dependents();                  // the next kernel may start its own set-up now
    if (warp == 0) {
        // ---------------- TMA producer: one stream of (tile, K block) pairs through the stage ring.  The weights do
        // not depend on the kernels before this one: the first ring of weight tiles is requested before the wait for
        // those kernels, the activations after it.
        // The first ring of the first tile is requested by one lane per stage, so that the requests go out together
        // (a single thread needs some hundred clocks per request, and the activations' requests sit on the critical path
        // right after the wait).
        const TileCoord c0 = tile_coord<(S::RECV_BYTES > 0)>(g, blockIdx.x, BN);
        const int early = (blockIdx.x < n_tiles_total) ? min(c0.n_kb, S::STAGES) : 0;
        if (lane < early) {
            mbar_expect_tx(full_bar(lane), S::STAGE_BYTES);
            tma_load_2d(a_base + lane * G_A_BYTES, &map_w, (c0.kb_begin + lane) * G_BK, c0.m0, full_bar(lane));
        }
        if (clustered) cluster_sync_all();       // every block's barriers exist before any block arrives on another's
        grid_dependency_wait();
        if (lane < early) tma_load_2d(b_base + lane * S::B_BYTES, &map_x, (c0.kb_begin + lane) * G_BK, c0.n0, full_bar(lane));
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < n_tiles_total && alive; t += gridDim.x) {
                const TileCoord c = tile_coord<(S::RECV_BYTES > 0)>(g, t, BN);
                int i = 0;
                if (it == 0) {
                    i = early;
                    it = early;
                }
                for (; i < c.n_kb; ++i, ++it) {
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, g.status, 1)) { alive = false; break; }
                    mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                    const int k = (c.kb_begin + i) * G_BK;
                    tma_load_2d(a_base + s * G_A_BYTES, &map_w, k, c.m0, full_bar(s));
                    tma_load_2d(b_base + s * S::B_BYTES, &map_x, k, c.n0, full_bar(s));
                }
            }
        }
    } else if (warp <= S::ISSUERS) {
        // ---------------- MMA issuers: tile j accumulates in buffer j % 2 (of each issuer) once the epilogue has emptied
        // it; issuer u takes the tile's K steps u, u + ISSUERS, ...
        if (clustered) cluster_sync_all();
        if (lane == 0) {
            constexpr unsigned idesc = umma_idesc(BN);
            const int u = warp - 1;
            int it = 0, j = 0;
            bool ok = true;
            int total_it = 0;                  // K steps of all of this block's tiles: a stage is handed back only if needed again
            for (int t = blockIdx.x; t < n_tiles_total; t += gridDim.x) total_it += tile_coord<(S::RECV_BYTES > 0)>(g, t, BN).n_kb;
            for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++j) {
                const TileCoord c = tile_coord<(S::RECV_BYTES > 0)>(g, t, BN);
                const int buf = j & 1;
                ok = mbar_wait(acc_empty_bar(buf), (((unsigned)j >> 1) & 1u) ^ 1u, g.status, 2);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned d_tmem = tmem_base + (unsigned)((u * 2 + buf) * S::ACC_COLS);
                // K steps are dealt out by their number in the block's whole sequence of steps, not by their place in the
                // tile: a stage's barrier is then waited on by one thread only, in the order of its phases (a parity wait
                // cannot tell a phase from the one two before it)
                bool first = true;
                for (int i = 0; i < c.n_kb; ++i, ++it) {
                    if (it % S::ISSUERS != u) continue;
                    const int s = it % S::STAGES;
                    const unsigned phase = (it / S::STAGES) & 1;
                    ok = mbar_wait(full_bar(s), phase, g.status, 2);
                    if (!ok) break;
                    if (stamps != nullptr && it == 0) stamps[2] = global_ns();            // first tiles have landed
                    tcgen05_fence_after();
                    const unsigned long long a_desc = umma_desc_sw128(a_base + s * G_A_BYTES);
                    const unsigned long long b_desc = umma_desc_sw128(b_base + s * S::B_BYTES);
#pragma unroll
                    for (int k = 0; k < G_BK / 16; ++k) {
                        // 16 elements = 32 bytes further along K inside the swizzle span: +2 in address/16 units
                        tcgen05_mma_f16(d_tmem, a_desc + 2ull * k, b_desc + 2ull * k, idesc, (!first || k > 0) ? 1u : 0u);
                    }
                    first = false;
                    if (it + S::STAGES < total_it) tcgen05_commit(empty_bar(s));      // the stage is free once these products have read it
                }
                if (!ok) break;
                if (stamps != nullptr && j == 0 && u == 0) stamps[3] = global_ns();       // first tile's last product issued
                // arrives when every product this thread has issued is done (at once if it had no K step in this tile)
                if (!first) tcgen05_commit(acc_full_bar(buf));
                else mbar_arrive(acc_full_bar(buf));
            }
        }
    } else {
        // ---------------- epilogue: warp q of a group reads tensor-memory lanes 32q .. 32q+31; the groups share out
        // the tile's tokens
        const int q = warp & 3;
        const int eg = (warp - 1 - S::ISSUERS) >> 2;
        const int et = threadIdx.x - 32 * (1 + S::ISSUERS);            // 0 .. 128*EG-1
        constexpr int COLS_PER_GROUP = BN / EG;
        if (clustered) cluster_sync_all();
        grid_dependency_wait();                // positions, page lists and the output buffers may come from earlier kernels
        // QKV through shared memory: when a warp's 32 rows are 16 rotation pairs of one head (head sizes in steps of 32)
        // and everything is bfloat16 and 16-byte aligned, results leave in 16-byte stores
        const bool qkv_fast = qkv_epilogue(EPI) && g.out_dtype == MLC_DTYPE_BF16 && (g.hd & 31) == 0 &&
                              ((((uintptr_t)g.out) | ((uintptr_t)g.cache.k_pool) | ((uintptr_t)g.cache.v_pool)) & 15) == 0 &&
                              (g.cache.entry_offset & 7) == 0;
        int j = 0, it_done = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles_total && ok; t += gridDim.x, ++j) {
            const TileCoord c = tile_coord<(S::RECV_BYTES > 0)>(g, t, BN);
            const int m0 = c.m0, n0 = c.n0, split = c.split;
            const int buf = j & 1;
            if (qkv_epilogue(EPI)) {
                for (int tt = et; tt < BN; tt += 128 * EG) {
                    int p = 0;
                    long long off = 0;
                    if (n0 + tt < g.n_tok) {
                        p = __ldg(g.positions + n0 + tt);
                        if (g.kv_heads > 0) off = paged_offset(g.cache, __ldg(g.tok_seq + n0 + tt), p, 0);
                    }
                    tok_pos[tt] = p;
                    tok_off[tt] = off;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(128 * EG) : "memory");          // the epilogue warps only
                if (S::ROPE_BYTES > 0 && qkv_fast) {
                    // cos and sin of this warp's 16 rotation pairs for its group's tokens, fetched while the products run
                    const int row0 = m0 + q * 32;
                    const int head0 = row0 / g.hd, i0 = (row0 % g.hd) >> 1, half = g.hd >> 1;
                    if (row0 < g.n_out && head0 < g.q_heads + g.kv_heads && g.rope != nullptr) {
                        float2* rs = reinterpret_cast<float2*>(smem_generic + rope_off) + (eg * 4 + q) * COLS_PER_GROUP * 16;
                        // eight loads in flight per lane: the loop is a chain of memory latencies otherwise
                        constexpr int PER_LANE = COLS_PER_GROUP * 16 / 32, BATCH = PER_LANE < 8 ? PER_LANE : 8;
#pragma unroll 1
                        for (int it = 0; it < PER_LANE; it += BATCH) {
                            float2 cs[BATCH];
#pragma unroll
                            for (int u = 0; u < BATCH; ++u) {
                                const int idx = lane + 32 * (it + u);
                                const int tt = eg * COLS_PER_GROUP + (idx >> 4);
                                cs[u] = make_float2(1.0f, 0.0f);
                                if (n0 + tt < g.n_tok)
                                    cs[u] = __ldg(g.rope + (long long)min(tok_pos[tt], g.rope_positions - 1) * half + i0 + (idx & 15));
                            }
#pragma unroll
                            for (int u = 0; u < BATCH; ++u) rs[lane + 32 * (it + u)] = cs[u];
                        }
                    }
                    __syncwarp();
                }
            }
            ok = mbar_wait(acc_full_bar(buf), ((unsigned)j >> 1) & 1u, g.status, 3);
            if (!ok) break;
            tcgen05_fence_after();
            if (stamps != nullptr && et == 0 && j == 0) { stamps[4] = global_ns(); stamps[6] = -clock64(); }
            const unsigned d_tmem = tmem_base + (unsigned)(buf * S::ACC_COLS);
            // issuers that had a K step in this tile: steps it0 .. it0 + n_kb - 1 of the block's sequence, dealt out in turn
            const int it0 = it_done;
            it_done += c.n_kb;
            const int row = m0 + q * 32 + lane;
            const float bias_row = (qkv_epilogue(EPI) && g.bias != nullptr && row < g.n_out) ? __ldg(g.bias + row) : 0.0f;
            // SiLU epilogue through shared memory: bfloat16 output, a full 16-output group inside the matrix, aligned rows
            const bool silu_staged = EPI == EPI_SILU_MUL && g.out_dtype == MLC_DTYPE_BF16 && ((g.n_out >> 1) & 7) == 0 &&
                                     (m0 + q * 32 + 32 <= g.n_out) && ((((uintptr_t)g.out) & 15) == 0);
            bf16* stage = reinterpret_cast<bf16*>(smem_generic + staging_off) + (eg * 4 + q) * COLS_PER_GROUP * 16;
#pragma unroll (qkv_epilogue(EPI) ? 2 : 1)
            for (int c0 = eg * COLS_PER_GROUP; c0 < (eg + 1) * COLS_PER_GROUP; c0 += 16) {
                float v[16];
                if (S::ISSUERS == 1) tmem_load16(d_tmem + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
                if (S::ISSUERS > 1) {
                    bool have = false;
#pragma unroll
                    for (int u = 0; u < S::ISSUERS; ++u) {
                        const int first_step = it0 + ((u - it0 % S::ISSUERS) + S::ISSUERS) % S::ISSUERS;
                        if (first_step < it0 + c.n_kb) {                // the same for the whole block
                            float w[16];
                            tmem_load16(d_tmem + (unsigned)(u * 2 * S::ACC_COLS) + ((unsigned)(q * 32) << 16) + (unsigned)c0, w);
#pragma unroll
                            for (int e = 0; e < 16; ++e) v[e] = have ? v[e] + w[e] : w[e];
                            have = true;
                        }
                    }
                }
                if (S::RECV_BYTES > 0 && clustered) {
                    // this warp's 32 rows x 16 tokens of partial sums go to the block that owns the rows; that block's
                    // warp adds up what the cluster's blocks sent, in the order of their ranks
                    const unsigned n_blocks = (unsigned)g.n_splits, rank = cluster_rank();
                    const unsigned per_owner = 4u / n_blocks;                      // warps (quarters of the tile's rows) a block owns
                    const unsigned owner = (unsigned)q / per_owner, mine_q = (unsigned)q % per_owner;
                    const unsigned recv_local = base + recv_off;
                    const unsigned dst = cluster_map(recv_local + (((rank * per_owner + mine_q) * 32u + (unsigned)lane) << 6), owner);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 16u * u), "f"(v[4 * u]), "f"(v[4 * u + 1]),
                                     "f"(v[4 * u + 2]), "f"(v[4 * u + 3]) : "memory");
                    mbar_arrive_remote(cluster_map(recv_bar, owner));
                    if (owner != rank) continue;                    // another block finishes these rows
                    ok = mbar_wait_cluster(recv_bar, 0u, g.status, 3);
                    if (!ok) break;
                    const float4* mine = reinterpret_cast<const float4*>(smem_generic + recv_off) + ((mine_q * 32 + lane) << 2);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float4 sum = mine[u];
                        for (unsigned r = 1; r < n_blocks; ++r) {
                            const float4 x = mine[(r * per_owner * 32 << 2) + u];
                            sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
                        }
                        v[4 * u] = sum.x; v[4 * u + 1] = sum.y; v[4 * u + 2] = sum.z; v[4 * u + 3] = sum.w;
                    }
                }
                if (EPI == EPI_ADD) {
                    if (row < g.n_out) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const int tok = n0 + c0 + jj;
                            if (tok < g.n_tok) atomicAdd((float*)g.out + (long long)tok * g.n_out + row, v[jj]);
                        }
                    }
                } else if (EPI == EPI_STORE) {
                    if (row < g.n_out) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const int tok = n0 + c0 + jj;
                            if (tok < g.n_tok) {
                                const long long idx = (long long)split * g.split_stride + (long long)tok * g.n_out + row;
                                if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, v[jj]);
                                else store_out<bf16>(g.out, idx, v[jj]);
                            }
                        }
                    }
                } else if (EPI == EPI_SILU_MUL) {
                    // even lane: gate_j, odd lane: up_j, j = row / 2
                    const int half_out = g.n_out >> 1;
                    if (silu_staged) {
                        // Two tokens per step so that every lane produces a value: the even lane of a pair takes
                        // token j (its own gate, the neighbour's up), the odd lane token j+1.  Results go to a
                        // per-warp staging tile [token][16 outputs] in shared memory and leave in 16-byte stores.
                        const int cl = c0 - eg * COLS_PER_GROUP;
#pragma unroll
                        for (int jj = 0; jj < 16; jj += 2) {
                            const float send = (lane & 1) ? v[jj] : v[jj + 1];
                            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                            const float gate = (lane & 1) ? recv : v[jj];
                            const float up = (lane & 1) ? v[jj + 1] : recv;
                            const float act = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                            stage[(cl + jj + (lane & 1)) * 16 + (lane >> 1)] = __float2bfloat16_rn(act);
                        }
                    } else {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const float other = __shfl_xor_sync(0xffffffffu, v[jj], 1);
                            const int tok = n0 + c0 + jj;
                            if ((lane & 1) == 0 && row < g.n_out && tok < g.n_tok) {
                                const float gate = v[jj], up = other;
                                const float act = gate * (1.0f / (1.0f + expf(-gate))) * up;
                                const long long idx = (long long)tok * half_out + (row >> 1);
                                if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, act);
                                else store_out<bf16>(g.out, idx, act);
                            }
                        }
                    }
                } else {
                    // QKV: stored row order inside a head is (0, hd/2, 1, hd/2+1, ...): even lane holds
                    // dim i = (row % hd) / 2, its odd neighbour dim i + hd/2.  Positions and cache offsets
                    // of the tile's tokens were put in shared memory while the products ran.
                    const int hd = g.hd, half = hd >> 1;
                    if (qkv_fast) {
                        const int row0 = m0 + q * 32;
                        if (row0 < g.n_out) {                       // n_out is a multiple of 32 here: the warp's rows all exist
                            const int head = row0 / hd, i0 = (row0 % hd) >> 1;
                            const bool second = (lane & 1) != 0;
                            const float b = bias_row;
                            const bool rotate = head < g.q_heads + g.kv_heads && g.rope != nullptr;
                            const bool is_q = head < g.q_heads;
                            const bool is_k = !is_q && head < g.q_heads + g.kv_heads;
                            const int kvh = is_k ? head - g.q_heads : head - g.q_heads - g.kv_heads;
                            bf16* st = reinterpret_cast<bf16*>(smem_generic + staging_off) + (eg * 4 + q) * 1024 + ((c0 >> 4) & 1) * 512;   // [16 tokens][32], two in turn
                            const float2* rs = reinterpret_cast<const float2*>(smem_generic + rope_off) +
                                               (eg * 4 + q) * COLS_PER_GROUP * 16 + (c0 - eg * COLS_PER_GROUP) * 16 + (lane >> 1);
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj) {
                                float2 cs = make_float2(1.0f, 0.0f);
                                if (rotate) {
                                    if (S::ROPE_BYTES > 0) cs = rs[jj * 16];
                                    else if (n0 + c0 + jj < g.n_tok)
                                        cs = __ldg(g.rope + (long long)min(tok_pos[c0 + jj], g.rope_positions - 1) * half + i0 + (lane >> 1));
                                }
                                const float mine = v[jj] + b;
                                const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                                const float y = second ? (other * cs.y + mine * cs.x) : (mine * cs.x - other * cs.y);
                                st[jj * 32 + (lane & 1) * 16 + (lane >> 1)] = __float2bfloat16_rn(y);     // dims i0.., then i0 + hd/2..
                            }
                            __syncwarp();
                            bf16* dst_base = is_q ? (bf16*)g.out : (bf16*)(is_k ? g.cache.k_pool : g.cache.v_pool);
#pragma unroll
                            for (int k = 0; k < 2; ++k) {            // 16 tokens x two runs of 32 bytes = 64 pieces of 16 bytes
                                const int id = lane + 32 * k;
                                const int jj = id >> 2, run = (id >> 1) & 1, sub = id & 1;
                                const int tt = c0 + jj;
                                if (n0 + tt < g.n_tok) {
                                    const long long at = is_q ? ((long long)(n0 + tt) * g.q_heads + head) * hd
                                                              : tok_off[tt] + (long long)kvh * g.cache.page_size * hd;
                                    *reinterpret_cast<uint4*>(dst_base + at + run * half + i0 + sub * 8) =
                                        *reinterpret_cast<const uint4*>(st + jj * 32 + run * 16 + sub * 8);
                                }
                            }
                            // no barrier here: the next 16 tokens go to the other staging tile, and the barrier after
                            // their writes orders this tile's reads before its next writes
                        }
                        continue;
                    }
                    const int head = row / hd, within = row % hd;
                    const int i = within >> 1;
                    const bool second = (within & 1) != 0;
                    const int d = second ? i + half : i;
                    const bool row_ok = row < g.n_out;
                    const float b = (g.bias != nullptr && row_ok) ? __ldg(g.bias + row) : 0.0f;
                    const bool rotate = head < g.q_heads + g.kv_heads && g.rope != nullptr;
                    const bool is_q = head < g.q_heads;
                    const bool is_k = !is_q && head < g.q_heads + g.kv_heads;
                    const int kvh = is_k ? head - g.q_heads : head - g.q_heads - g.kv_heads;
                    const long long head_off = (long long)kvh * g.cache.page_size * hd + d;
                    // rotation factors of the 16 tokens first (independent loads), then arithmetic and stores
                    float2 cs[16];
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const int tt = c0 + jj;
                        cs[jj] = make_float2(1.0f, 0.0f);
                        if (rotate && row_ok && n0 + tt < g.n_tok)
                            cs[jj] = __ldg(g.rope + (long long)min(tok_pos[tt], g.rope_positions - 1) * half + i);
                    }
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const int tt = c0 + jj;
                        const float mine = v[jj] + b;
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        // first half: x0·c − x1·s; second half: x0·s + x1·c, with (x0, x1) = (dim i, dim i + hd/2)
                        const float y = second ? (other * cs[jj].y + mine * cs[jj].x) : (mine * cs[jj].x - other * cs[jj].y);
                        if (!row_ok || n0 + tt >= g.n_tok) continue;
                        if (is_q) {
                            const long long idx = ((long long)(n0 + tt) * g.q_heads + head) * hd + d;
                            if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, y);
                            else store_out<bf16>(g.out, idx, y);
                        } else {
                            void* pool = is_k ? g.cache.k_pool : g.cache.v_pool;
                            const long long off = tok_off[tt] + head_off;
                            if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(pool, off, y);
                            else store_out<bf16>(pool, off, y);
                        }
                    }
                }
            }
            if (stamps != nullptr && et == 0) stamps[7] = clock64();
            // the accumulator has been read: the tensor cores may fill it again
            tcgen05_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty_bar(buf)) : "memory");
            if (EPI == EPI_SILU_MUL && silu_staged) {
                __syncwarp();
                const int half_out = g.n_out >> 1;
                for (int tl = lane; tl < COLS_PER_GROUP; tl += 32) {
                    const int tok = n0 + eg * COLS_PER_GROUP + tl;
                    if (tok < g.n_tok) {
                        const uint4* src = reinterpret_cast<const uint4*>(stage + tl * 16);
                        uint4* dst = reinterpret_cast<uint4*>((bf16*)g.out + (long long)tok * half_out + (m0 >> 1) + q * 16);
                        dst[0] = src[0];
                        dst[1] = src[1];
                    }
                }
                __syncwarp();                  // the staging tile is free for the warp's next tile
            }
            if (qkv_epilogue(EPI)) asm volatile("bar.sync 1, %0;" ::"n"(128 * EG) : "memory");   // before the next tile's positions
        }
        if (stamps != nullptr && et == 0) stamps[5] = global_ns();                       // epilogues done
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
// A row-major bfloat16 matrix [rows][cols] read in boxes of box_rows x 64 columns.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    return cached_map_2d(map, ptr, rows, cols, G_BK, box_rows);
}

template <int BN, int EPI>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, int n_sms, cudaStream_t s) {
    using S = GemmShape<BN, EPI>;
    static_assert(S::SMEM_BYTES <= 227 * 1024, "shared memory of a block");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // persistent blocks: one per SM at most, each walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...
    const long long tiles = (long long)g.m_tiles * g.n_tiles * g.n_splits;
    if (g.cluster_split) {
        // one tile and one K range per block; the n_splits blocks of a tile are neighbours and form a cluster
        if (S::RECV_BYTES == 0 || tiles > 0x7fffffffll) return MLC_ERR_BAD_SIZE;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)tiles);
        cfg.blockDim = dim3(S::THREADS);
        cfg.dynamicSmemBytes = (size_t)S::SMEM_BYTES;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)g.n_splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, EPI>, mw, mx, g);
        return e == cudaSuccess ? 0 : (int)e;
    }
    const unsigned blocks = (unsigned)(tiles < n_sms ? tiles : n_sms);
    cudaError_t e = launch_pdl(gemm_tcgen05_kernel<BN, EPI>, dim3(blocks), dim3(S::THREADS), (size_t)S::SMEM_BYTES, s, mw, mx, g);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int EPI>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, int n_sms, cudaStream_t s) {
    switch (bn) {
        case 16: return launch_gemm<16, EPI>(mw, mx, g, n_sms, s);
        case 32: return launch_gemm<32, EPI>(mw, mx, g, n_sms, s);
        case 64: return launch_gemm<64, EPI>(mw, mx, g, n_sms, s);
        case 128: return launch_gemm<128, EPI>(mw, mx, g, n_sms, s);
        case 256: return launch_gemm<256, EPI>(mw, mx, g, n_sms, s);
    }
    return MLC_ERR_BAD_SIZE;
}

}  // namespace mlc

using namespace mlc;

// How many clusters of `size` (2 or 4) blocks of the few-token Q/K/V product the GPU holds at once; 0 if such clusters
// cannot be launched.  A tile count above this number runs in rounds.
extern "C" int mlc_gemm_qkv_clusters_resident(int size) {
    static int cached[5] = {0, 0, 0, 0, 0};
    static bool known[5] = {false, false, false, false, false};
    if (size != 2 && size != 4) return 0;
    if (!known[size]) {
        using S = GemmShape<16, EPI_QKV_CLUSTER>;
        int n = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<16, EPI_QKV_CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)size);
            cfg.blockDim = dim3(S::THREADS);
            cfg.dynamicSmemBytes = (size_t)S::SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)size;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_kernel<16, EPI_QKV_CLUSTER>, &cfg) != cudaSuccess) n = 0;
        }
        (void)cudaGetLastError();
        cached[size] = n;
        known[size] = true;
    }
    return cached[size];
}

// x: bfloat16 [n_tok][K]; w: bfloat16 [n_out][K] (K a multiple of 8, both 16-byte aligned).
// epilogue 0: out [n_splits][n_tok][n_out] (float32 or bfloat16): with n_splits > 1 the K range is shared out over
// blocks and each leaves its partial sums in its own slice for the consumer to add; 1: out [n_tok][n_out/2],
// n_splits must be 1;
// 2: out = q [n_tok][q_heads*hd], k and v go to the cache, n_splits 1, or 2 or 4 with block_tokens 16 (the K range
// shared out over the blocks of a cluster, which merge before the epilogue); 3: adds into out (float32
// [n_tok][n_out]) atomically, any n_splits.
// block_tokens: 16, 32, 64, 128 or 256.  status: one int on the device, 0 before the call; a bounded
// wait that ran out leaves 1 (loader), 2 (tensor cores) or 3 (epilogue) there.  timing: null, or
// [blocks][8] uint64 that receive nanosecond stamps of each block's phases.  n_sms: blocks to launch at most.
extern "C" int mlc_gemm_tcgen05(const void* x, const void* w, void* out, int out_dtype, int n_tok, int n_out, int K,
                                int block_tokens, int n_splits, int epilogue, int* status, unsigned long long* timing,
                                int n_sms, const float* bias, const int* positions, const int* tok_seq,
                                const void* rope_table, int rope_positions, int q_heads, int kv_heads, int hd,
                                void* k_pool, void* v_pool, const int* page_table, long long entry_offset,
                                int pages_per_seq, int page_size, void* stream) {
    if (n_tok <= 0 || n_out <= 0) return 0;
    if (K <= 0 || (K & 7) || (((uintptr_t)x | (uintptr_t)w) & 15)) return MLC_ERR_BAD_SIZE;
    if (out_dtype != MLC_DTYPE_F32 && out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    // Q/K/V: 2 or 4 blocks of a cluster may share a tile's K range (16-token tiles only)
    const bool cluster_split = epilogue == EPI_QKV && n_splits > 1;
    if (cluster_split && !((n_splits == 2 || n_splits == 4) && block_tokens == 16)) return MLC_ERR_BAD_SIZE;
    if (n_splits < 1 || (epilogue != EPI_STORE && epilogue != EPI_ADD && !cluster_split && n_splits != 1) || status == nullptr) return MLC_ERR_BAD_SIZE;
    if (epilogue == EPI_ADD && out_dtype != MLC_DTYPE_F32) return MLC_ERR_BAD_DTYPE;
    if (n_sms < 1) return MLC_ERR_BAD_SIZE;
    GemmArgs g{};
    g.out = out;
    g.out_dtype = out_dtype;
    g.n_out = n_out;
    g.n_tok = n_tok;
    g.k_blocks = (K + G_BK - 1) / G_BK;
    g.k_blocks_per_split = (g.k_blocks + n_splits - 1) / n_splits;
    if ((long long)(n_splits - 1) * g.k_blocks_per_split >= g.k_blocks) return MLC_ERR_BAD_SIZE;   // an empty split
    g.split_stride = (long long)n_tok * n_out;
    g.status = status;
    g.timing = timing;
    g.m_tiles = (n_out + G_BM - 1) / G_BM;
    g.n_tiles = (n_tok + block_tokens - 1) / block_tokens;
    g.n_splits = n_splits;
    g.cluster_split = cluster_split ? 1 : 0;
    if (epilogue == EPI_SILU_MUL && (n_out & 1)) return MLC_ERR_BAD_SIZE;
    if (epilogue == EPI_QKV) {
        if (hd <= 0 || (hd & 1) || n_out != (q_heads + 2 * kv_heads) * hd || positions == nullptr) return MLC_ERR_BAD_SIZE;
        if (kv_heads > 0 && (tok_seq == nullptr || k_pool == nullptr || v_pool == nullptr || page_table == nullptr)) return MLC_ERR_BAD_SIZE;
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
    CUtensorMap mw, mx;
    int rc = make_map(&mw, w, n_out, K, G_BM);
    if (rc) return rc;
    rc = make_map(&mx, x, n_tok, K, block_tokens);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == EPI_STORE) return dispatch_bn<EPI_STORE>(block_tokens, mw, mx, g, n_sms, s);
    if (epilogue == EPI_SILU_MUL) return dispatch_bn<EPI_SILU_MUL>(block_tokens, mw, mx, g, n_sms, s);
    if (epilogue == EPI_QKV && cluster_split) return launch_gemm<16, EPI_QKV_CLUSTER>(mw, mx, g, n_sms, s);
    if (epilogue == EPI_QKV) return dispatch_bn<EPI_QKV>(block_tokens, mw, mx, g, n_sms, s);
    if (epilogue == EPI_ADD) return dispatch_bn<EPI_ADD>(block_tokens, mw, mx, g, n_sms, s);
    return MLC_ERR_UNSUPPORTED;
}

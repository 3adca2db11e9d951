// Prompt attention on the fifth-generation tensor cores: softmax(q·kᵀ·scale)·v of many tokens over
// a paged bfloat16 cache (src/ops.cpp:143-196 gives the arithmetic), scores and outputs accumulated in
// tensor memory, operands staged in shared memory by TMA.
//
// A block owns 128 rows of one key/value head: the group's query heads of 128 / group successive
// tokens (one row per token and head, so keys are read once for the whole group), and walks the
// keys the rows may see in tiles of 64, which is one page of the cache.  Roles:
//     warp 0     one thread issues the TMA loads: the query rows once, then a ring of K and V pages;
//     warp 1     allocates tensor memory; one thread issues tcgen05.mma: S_j = Q·K_jᵀ into one of two
//                score buffers, and O += P_j·V_j (V is the MN-major operand, read as the cache holds it);
//     warps 2-9  two threads per row (each 32 of a tile's keys): read the row's 64 scores from tensor memory, mask where the tile
//                meets the diagonal, a window's edge or padding rows, keeps the running maximum and sum
//                in float32, writes P_j = exp2(s·scale·log2e − m) as bfloat16 into shared memory for the
//                tensor cores.  The output accumulates in tensor memory; when a row's maximum rises by more than
//                2^8 the row's thread rescales its lane of the output there before O_j is added.
// The tensor cores compute S_{j+1} and O_j while the rows work on tile j.  With a head size of 64 two
// blocks share an SM, so one block's exponentials overlap the other's products.
//
// Pages are handed out dirty.  Keys beyond a row's range give scores that are replaced, not multiplied; values
// beyond the sequence's last key would meet probabilities of exactly zero, but 0 x NaN is NaN, so the rows of
// the last page's V tile that lie beyond the sequence are zeroed in shared memory before the product reads them.
//
// Every wait on an mbarrier is bounded by a clock; a wait that runs out records a code in `status`
// (11 loader, 12 tensor cores, 13 softmax rows), the block skips its stores, frees its tensor memory
// and returns.
#include "tcgen05.cuh"

#ifndef MLC_HEAD_DIM
#define MLC_HEAD_DIM 64
#endif

#if MLC_HEAD_DIM == 64 || MLC_HEAD_DIM == 128
#define MLC_ATTENTION_TCGEN05 1
#else
#define MLC_ATTENTION_TCGEN05 0
#endif

namespace mlc {

struct TcAttnArgs {
    void* out;                  // bfloat16 [tokens][q_heads*hd]
    const int* cu_seqlens;      // [n_seqs + 1] first token of each sequence in the step
    const int* start_pos;       // [n_seqs] position of each sequence's first token of the step
    const int* page_table;      // [n_seqs][pages_per_seq]
    int pages_per_seq;
    int q_heads, kv_heads, group;
    int heads_per_block, tokens_per_block, head_chunks;
    int window;
    int n_splits;               // blocks that share out a row tile's keys: one cluster, merged through distributed shared memory
    float scale_log2;
    int* status;
    long long* timing;          // optional [blocks][16] clock cycles spent in each phase by the first softmax warp (0-7)
                                // and by the issuing thread (8-15), for tuning; or null
};

#if MLC_ATTENTION_TCGEN05

constexpr int A_HD = MLC_HEAD_DIM;
constexpr int A_BM = 128;                              // rows of a block
constexpr int A_BN = 64;                               // keys of a tile: one page
constexpr int A_KB = A_HD / 64;                        // 64-element spans of the head size
constexpr int A_STAGES = 3;
constexpr int A_Q_BYTES = A_KB * A_BM * 128;
constexpr int A_TILE_BYTES = A_KB * A_BN * 128;        // one K or V page of one head
constexpr int A_P_BYTES = A_BM * 128;
constexpr int A_BAR_BYTES = 256 + 1024 + 1024;         // barriers, the row sums' exchange [2][128] floats, a split's (max, sum) [128][2]
constexpr int A_PART_STRIDE = A_HD + 4;                // floats between rows of a split's partial output (padded against bank conflicts)
static_assert(A_BM * A_PART_STRIDE * 4 <= 2 * 3 * (A_HD / 64) * 64 * 128, "a split's partial output reuses the K and V stages");
constexpr int A_THREADS = 64 + 256;
constexpr int A_SMEM_BYTES = A_Q_BYTES + 2 * A_STAGES * A_TILE_BYTES + 2 * A_P_BYTES + A_BAR_BYTES + 1024 /* alignment slack */;
constexpr int A_TMEM_COLS = 256;                       // two score buffers of 64 columns, the output's A_HD
static_assert(2 * A_BN + A_HD <= A_TMEM_COLS, "tensor memory of a block");
constexpr int A_BLOCKS_PER_SM = (A_HD == 64) ? 2 : 1;
static_assert(A_SMEM_BYTES * A_BLOCKS_PER_SM <= 226 * 1024, "shared memory of the blocks of one SM");

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(A_THREADS, A_BLOCKS_PER_SM)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, TcAttnArgs a) {
    const int t_entry = (int)clock();
    const unsigned long long g_entry = global_ns();
    // ---- which rows: heavy blocks (late tokens see the most keys) first
    // blocks are handed out x first: every sequence's and head's last rows before anyone's earlier rows
    const int heads_y = a.kv_heads * a.head_chunks;
    const int split = blockIdx.x % a.n_splits, xh = blockIdx.x / a.n_splits;      // the splits of a row tile are one cluster
    const int b = xh / heads_y;
    const int kvh = (xh % heads_y) / a.head_chunks, chunk = xh % a.head_chunks;
    const int tok0 = (gridDim.y - 1 - blockIdx.y) * a.tokens_per_block;

    extern __shared__ unsigned char smem_dyn[];
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    const unsigned q_base = base;
    const unsigned k_base = q_base + A_Q_BYTES;
    const unsigned v_base = k_base + A_STAGES * A_TILE_BYTES;
    const unsigned p_base = v_base + A_STAGES * A_TILE_BYTES;
    constexpr unsigned v_off = A_Q_BYTES + A_STAGES * A_TILE_BYTES;
    constexpr unsigned p_off = A_Q_BYTES + 2 * A_STAGES * A_TILE_BYTES;
    const unsigned bar_base = p_base + 2 * A_P_BYTES;
    constexpr unsigned bar_off = p_off + 2 * A_P_BYTES;
    auto k_full = [&](int s) { return bar_base + 8u * s; };
    auto v_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (8 + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (26 + s); };
    auto s_full = [&](int i) { return bar_base + 8u * (12 + i); };
    auto p_full = [&](int i) { return bar_base + 8u * (16 + i); };
    auto o_full = [&](int i) { return bar_base + 8u * (20 + i); };       // O_j complete: barrier j & 1
    const unsigned q_full = bar_base + 8u * 24;
    const unsigned tmem_slot = bar_base + 8u * 25;
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + bar_off + 8 * 25);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_empty(s), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full(i), 1);
            mbar_init(p_full(i), 256);
        }
        mbar_init(q_full, 1);
        mbar_init(o_full(0), 1);
        mbar_init(o_full(1), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((unsigned)A_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_base = *tmem_slot_ptr;
    grid_launch_dependents();
    grid_dependency_wait();                    // the queries and the step's keys come from the kernel before

    const int seq_tok0 = a.cu_seqlens[b];
    const int q_len = a.cu_seqlens[b + 1] - seq_tok0;
    const int n_tok = min(a.tokens_per_block, q_len - tok0);          // <= 0: nothing to do for this block
    const int start = a.start_pos[b];
    const int p_first = start + tok0, p_last = start + tok0 + n_tok - 1;
    const int lo_block = (a.window > 0) ? max(0, p_first - a.window + 1) : 0;
    const bool active = n_tok > 0;                                   // the same for every block of a cluster
    const int tiles_all = active ? p_last / A_BN + 1 - lo_block / A_BN : 0;
    const int tiles_per_split = (tiles_all + a.n_splits - 1) / a.n_splits;
    const int tile_begin = lo_block / A_BN + split * tiles_per_split;
    const int n_tiles = max(0, min(tiles_per_split, tiles_all - split * tiles_per_split));
    const bool clustered = a.n_splits > 1 && active;
    auto cluster_sync = [&]() {
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    };
    const int* pages = a.page_table + (long long)b * a.pages_per_seq;
    const int seq_last = start + q_len - 1;                          // the sequence's last key

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0 && n_tiles > 0) {
            // a box is heads_per_block x tokens_per_block rows whatever part of it lies outside the tensor; rows of the
            // tile past the box are not written, and nothing reads their results
            mbar_expect_tx(q_full, (unsigned)(A_KB * a.heads_per_block * a.tokens_per_block * 128));
            for (int kb = 0; kb < A_KB; ++kb)
                tma_load_3d(q_base + kb * A_BM * 128, &map_q, kb * 64, kvh * a.group + chunk * a.heads_per_block,
                            seq_tok0 + tok0, q_full);
            // K_j is wanted one tile before V_j (the scores run a tile ahead), and its stage is free as soon as S_j is done:
            // the order is K_0, K_1, V_0, K_2, V_1, ...
            auto load_k = [&](int j, int page) -> bool {
                const int s = j % A_STAGES;
                if (!mbar_wait(k_empty(s), ((j / A_STAGES) & 1) ^ 1u, a.status, 11)) return false;
                const int row = (page * a.kv_heads + kvh) * A_BN;       // a missing page (-1) reads as zeros
                mbar_expect_tx(k_full(s), A_TILE_BYTES);
                for (int kb = 0; kb < A_KB; ++kb)
                    tma_load_2d(k_base + s * A_TILE_BYTES + kb * A_BN * 128, &map_k, kb * 64, row, k_full(s));
                return true;
            };
            auto load_v = [&](int j, int page) -> bool {
                const int s = j % A_STAGES;
                if (!mbar_wait(v_empty(s), ((j / A_STAGES) & 1) ^ 1u, a.status, 11)) return false;
                const int row = (page * a.kv_heads + kvh) * A_BN;
                mbar_expect_tx(v_full(s), A_TILE_BYTES);
                for (int kb = 0; kb < A_KB; ++kb)
                    tma_load_2d(v_base + s * A_TILE_BYTES + kb * A_BN * 128, &map_v, kb * 64, row, v_full(s));
                return true;
            };
            int page_v = __ldg(pages + tile_begin);                                     // page of tile j
            int page_k = (n_tiles > 1) ? __ldg(pages + tile_begin + 1) : 0;              // page of tile j + 1
            bool alive = load_k(0, page_v);
            for (int j = 0; j < n_tiles && alive; ++j) {
                const int page_next = (j + 2 < n_tiles) ? __ldg(pages + tile_begin + j + 2) : 0;
                if (j + 1 < n_tiles) alive = load_k(j + 1, page_k);
                if (alive) alive = load_v(j, page_v);
                page_v = page_k;
                page_k = page_next;
            }
        }
        if (clustered) {                       // every thread of the cluster meets at both barriers of the merge
            cluster_sync();
            cluster_sync();
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issuer
        if (lane == 0 && n_tiles > 0) {
            constexpr unsigned idesc_s = umma_idesc(A_BN);
            constexpr unsigned idesc_o = umma_idesc(A_HD, true);
            const bool stamp = a.timing != nullptr;
            int ph[6] = {0, 0, 0, 0, 0, 0}, t0 = 0, t1;
#define MLC_PHASE(k) if (stamp) { t1 = (int)clock(); ph[k] += t1 - t0; t0 = t1; }
            bool ok = mbar_wait(q_full, 0, a.status, 12);
            if (stamp) t0 = (int)clock();
            auto issue_scores = [&](int j) -> bool {
                const int s = j % A_STAGES, i = j & 1;
                if (!mbar_wait(k_full(s), (j / A_STAGES) & 1, a.status, 12)) return false;
                MLC_PHASE(0)                                   // waiting for K
                // the score buffer is free: the rows handed over P_{j-2} (seen in the last round) after reading S_{j-2}
                tcgen05_fence_after();
                const unsigned d = tmem_base + (unsigned)(i * A_BN);
#pragma unroll
                for (int kb = 0; kb < A_KB; ++kb) {
                    const unsigned long long qd = umma_desc_sw128(q_base + kb * A_BM * 128);
                    const unsigned long long kd = umma_desc_sw128(k_base + s * A_TILE_BYTES + kb * A_BN * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tcgen05_mma_f16(d, qd + 2ull * k, kd + 2ull * k, idesc_s, (kb > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(s_full(i));      // arrives when S_j and everything issued before it (O_{j-2} too) is complete
                MLC_PHASE(2)                                   // issuing S
                return true;
            };
            if (ok) ok = issue_scores(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    ok = issue_scores(j + 1);
                    if (!ok) break;
                }
                const int s = j % A_STAGES, i = j & 1;
                ok = mbar_wait(v_full(s), (j / A_STAGES) & 1, a.status, 12);
                MLC_PHASE(3)                                   // waiting for V
                ok = ok && mbar_wait(p_full(i), ((unsigned)j >> 1) & 1u, a.status, 12);      // P_j written, the output rescaled
                if (!ok) break;
                MLC_PHASE(4)                                   // waiting for P
                tcgen05_fence_after();
                const unsigned d = tmem_base + (unsigned)(2 * A_BN);
                const unsigned long long pd = umma_desc_sw128(p_base + i * A_P_BYTES);
                const unsigned long long vd = umma_desc_sw128_mn(v_base + s * A_TILE_BYTES, A_BN * 128);
#pragma unroll
                for (int k = 0; k < 4; ++k)      // 16 keys a step: 32 bytes along a row of P, two 8-key groups of V
                    tcgen05_mma_f16(d, pd + 2ull * k, vd + (unsigned long long)((2048u >> 4) * k), idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(o_full(i));
                MLC_PHASE(5)                                   // issuing O
            }
            if (stamp) {
                long long* dst = a.timing + 16ll * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)) + 8;
                for (int k = 0; k < 6; ++k) dst[k] = ph[k];
            }
#undef MLC_PHASE
        }
        if (clustered) {
            cluster_sync();
            cluster_sync();
        }
    } else if (active) {
        // ---------------- two threads per row: warps 2-5 take keys 0-31 of every tile and the first half of the output's
        // columns, warps 6-9 keys 32-63 and the second half.  Both read all 64 scores for the maximum, so they agree on
        // the scale without exchanging anything; only the row sums meet at the end.
        const int q4 = warp & 3;
        const int half = (warp - 2) >> 2;
        const int st_id = threadIdx.x - 64;                 // 0 .. 255
        const int r = q4 * 32 + lane;
        const int t = r / a.heads_per_block, hg = chunk * a.heads_per_block + r % a.heads_per_block;
        const bool row_ok = t < n_tok && hg < a.group && r < a.heads_per_block * a.tokens_per_block;
        // Rows that do not exist take the range of the block's last token: they then mask exactly when their neighbours
        // do, whatever lies in their part of the query tile, and nothing of theirs is stored.
        const int hi = start + tok0 + min(t, n_tok - 1);
        const int lo = (a.window > 0) ? max(0, hi - a.window + 1) : 0;
        const unsigned lane_base = (unsigned)(q4 * 32) << 16;
        // m is the maximum the row's probabilities and output are scaled by.  It follows the true maximum lazily: only
        // when a tile's maximum exceeds it by more than 8 (probabilities up to 2^8, harmless in float32 and bfloat16)
        // is the output in tensor memory rescaled, so that after the first tiles the rescaling almost never runs.
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        const bool stamp = a.timing != nullptr && warp == 2;      // the whole warp keeps time, so that it stays converged
        int ph[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t0 = 0, t1;        // 32-bit clocks: differences survive the wrap
#define MLC_PHASE(k) if (stamp) { t1 = (int)clock(); ph[k] += t1 - t0; t0 = t1; }
        if (stamp) t0 = (int)clock();
        const int t_role = t0;
        constexpr int O_COLS = A_HD / 2;                    // output columns of one thread
        const unsigned o_taddr = tmem_base + lane_base + (unsigned)(2 * A_BN + half * O_COLS);

        for (int j = 0; j < n_tiles; ++j) {
            const int i = j & 1;
            ok = mbar_wait(s_full(i), ((unsigned)j >> 1) & 1u, a.status, 13);
            if (!ok) break;
            MLC_PHASE(0)                                   // waiting for the scores
            tcgen05_fence_after();
            float s[32], u[32];                            // this thread's keys, and the other half's (for the maximum)
            tmem_load32(tmem_base + lane_base + (unsigned)(i * A_BN + half * 32), s);
            tmem_load32(tmem_base + lane_base + (unsigned)(i * A_BN + (half ^ 1) * 32), u);
            tcgen05_fence_before();
            if (threadIdx.x == 64) {
                // S_j is complete, and with it everything the issuing thread had issued before: O_{j-2}.  Their K and V
                // stages are free for the loader.
                mbar_arrive(k_empty(j % A_STAGES));
                if (j >= 2) mbar_arrive(v_empty((j - 2) % A_STAGES));
            }
            __syncwarp();
            MLC_PHASE(1)                                   // reading them

            const int key0 = (tile_begin + j) * A_BN;
            // decided for the warp as a whole: lanes that went separate ways here would run everything below twice
            if (!__all_sync(0xffffffffu, key0 + A_BN - 1 <= hi && key0 >= lo)) {
                const int ks = key0 + half * 32, ku = key0 + (half ^ 1) * 32;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    s[c] = (ks + c >= lo && ks + c <= hi) ? s[c] : -INFINITY;
                    u[c] = (ku + c >= lo && ku + c <= hi) ? u[c] : -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one of 64 links
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
                mx4[0] = fmaxf(mx4[0], fmaxf(s[c], u[c]));
                mx4[1] = fmaxf(mx4[1], fmaxf(s[c + 1], u[c + 1]));
                mx4[2] = fmaxf(mx4[2], fmaxf(s[c + 2], u[c + 2]));
                mx4[3] = fmaxf(mx4[3], fmaxf(s[c + 3], u[c + 3]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;   // the scale is positive
            const bool raise = mx > m + 8.0f;                         // false while nothing has been seen (-inf > -inf)
            const float m_new = raise ? mx : m;
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float corr = raise ? fast_exp2(m - m_use) : 1.0f;   // 0 when nothing was seen before
            m = m_new;
            float ls4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            unsigned pk[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float p0 = fast_exp2(fmaf(s[2 * c], a.scale_log2, -m_use));
                const float p1 = fast_exp2(fmaf(s[2 * c + 1], a.scale_log2, -m_use));
                ls4[(2 * c) & 3] += p0;
                ls4[(2 * c + 1) & 3] += p1;
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                pk[c] = *reinterpret_cast<unsigned*>(&h);
            }
            const float ls = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
            l = l * corr + ls;
            MLC_PHASE(2)                                   // mask, maximum, exponentials

            if (key0 + A_BN - 1 > seq_last) {
                // the tile reaches past the sequence's last key: zero those rows of V (whole 128-byte rows, so the
                // swizzle does not matter) once TMA has delivered the tile
                const int st = j % A_STAGES;
                ok = mbar_wait(v_full(st), (j / A_STAGES) & 1, a.status, 13);
                if (!ok) break;
                const int first = max(seq_last + 1 - key0, 0), n_rows = A_BN - first;
                for (int idx = st_id; idx < n_rows * 8 * A_KB; idx += 256) {
                    const int kb = idx / (n_rows * 8), rem = idx % (n_rows * 8);
                    *reinterpret_cast<uint4*>(smem_generic + v_off + st * A_TILE_BYTES + kb * A_BN * 128 + (first + rem / 8) * 128 +
                                              (rem % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            // the P buffer is free: O_{j-2}, which read it, was complete when S_j was
            unsigned char* prow = smem_generic + p_off + i * A_P_BYTES + r * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(prow + (((half * 4 + c) ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            fence_async_shared();
            MLC_PHASE(4)                                   // writing P

            if (j > 0 && __any_sync(0xffffffffu, raise)) {
                // Rescale this warp's part of the output before P_j·V_j is added to it; O_{j-1} must be complete.  (A parity
                // wait tells a barrier's phases k and k + 2 apart only if the barrier is known to be within one phase of k.
                // O_j completes barrier j & 1; this thread has read S_j, which was issued after O_{j-2}, and O_{j+1} cannot
                // be issued before this thread hands over P_{j+1}: so barrier (j-1) & 1 is at O_{j-1} or just before it.)
                ok = mbar_wait(o_full((j - 1) & 1), ((unsigned)(j - 1) >> 1) & 1u, a.status, 13);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < O_COLS; c0 += 32) {
                    float v[32];
                    tmem_load32(o_taddr + (unsigned)c0, v);
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] *= corr;
                    tmem_store32(o_taddr + (unsigned)c0, v);
                }
                tmem_store_wait();
                tcgen05_fence_before();
            }
            mbar_arrive(p_full(i));
            MLC_PHASE(5)                                   // rescaling
        }
        if (ok && n_tiles > 0) ok = mbar_wait(o_full((n_tiles - 1) & 1), ((unsigned)(n_tiles - 1) >> 1) & 1u, a.status, 13);
        MLC_PHASE(6)                                       // waiting for the last product
        if (stamp && lane == 0) {
            long long* dst = a.timing + 16ll * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
            for (int k = 0; k < 7; ++k) dst[k] = ph[k];
            dst[7] = n_tiles;
        }
#undef MLC_PHASE
        // the two halves of a row add up their sums
        float* l_part = reinterpret_cast<float*>(smem_generic + bar_off + 256);       // [2][128]
        l_part[half * 128 + r] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");                                 // the softmax warps only
        l += l_part[(half ^ 1) * 128 + r];
        tcgen05_fence_after();
        bf16* dst = (bf16*)a.out + ((long long)(seq_tok0 + tok0 + t) * a.q_heads + kvh * a.group + hg) * A_HD + half * O_COLS;
        float* part_o = reinterpret_cast<float*>(smem_generic + A_Q_BYTES);           // [128][A_PART_STRIDE], over the K and V stages
        float* part_ml = reinterpret_cast<float*>(smem_generic + bar_off + 256 + 1024);   // [128][2]
        if (clustered && split > 0) {
            // this block's share of the keys: leave (max, sum, unnormalised output) in shared memory for the first block.
            // The stages are free: every tile that was loaded has been multiplied.
#pragma unroll
            for (int c0 = 0; c0 < O_COLS; c0 += 32) {
                float v[32];
                if (n_tiles > 0) tmem_load32(o_taddr + (unsigned)c0, v);
                else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = 0.0f;
                }
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    *reinterpret_cast<float4*>(part_o + r * A_PART_STRIDE + half * O_COLS + c0 + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
            }
            if (half == 0) {
                part_ml[2 * r] = m;
                part_ml[2 * r + 1] = l;
            }
        }
        if (clustered) cluster_sync();
        if (!clustered || split == 0) {
            // merge the other blocks' shares (the first block always has tiles), normalise, store
            float scale_own = 1.0f, l_all = l;
            unsigned peer_o[3], peer_ml[3];
            float peer_f[3];
            const int n_peers = clustered ? a.n_splits - 1 : 0;
            if (n_peers > 0) {
                float m_all = m, mk[3], lk[3];
                const unsigned o_local = smem_u32(part_o), ml_local = smem_u32(part_ml);
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    mk[k] = -INFINITY;
                    lk[k] = 0.0f;
                    if (k >= n_peers) continue;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_o[k]) : "r"(o_local), "r"(k + 1));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer_ml[k]) : "r"(ml_local), "r"(k + 1));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mk[k]) : "r"(peer_ml[k] + 8u * r));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(lk[k]) : "r"(peer_ml[k] + 8u * r + 4u));
                    m_all = fmaxf(m_all, mk[k]);
                }
                const float m_ref = (m_all == -INFINITY) ? 0.0f : m_all;
                scale_own = fast_exp2(m - m_ref);
                l_all = l * scale_own;
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    peer_f[k] = fast_exp2(mk[k] - m_ref);                   // 0 for a block that saw nothing (or is not there)
                    l_all += lk[k] * peer_f[k];
                }
            }
            const float inv = 1.0f / l_all;
#pragma unroll
            for (int c0 = 0; c0 < O_COLS; c0 += 32) {
                float v[32];
                tmem_load32(o_taddr + (unsigned)c0, v);          // every lane of the warp takes part in the load
                if (n_peers > 0) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] *= scale_own;
#pragma unroll
                    for (int k = 0; k < 3; ++k) {
                        if (k >= n_peers) continue;
                        const unsigned base_k = peer_o[k] + 4u * (unsigned)(r * A_PART_STRIDE + half * O_COLS + c0);
#pragma unroll
                        for (int c = 0; c < 32; c += 4) {
                            float4 p;
                            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(p.x), "=f"(p.y), "=f"(p.z), "=f"(p.w) : "r"(base_k + 4u * c));
                            v[c] = fmaf(p.x, peer_f[k], v[c]);
                            v[c + 1] = fmaf(p.y, peer_f[k], v[c + 1]);
                            v[c + 2] = fmaf(p.z, peer_f[k], v[c + 2]);
                            v[c + 3] = fmaf(p.w, peer_f[k], v[c + 3]);
                        }
                    }
                }
                if (row_ok && ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        unsigned w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(v[c + 2 * e] * inv, v[c + 2 * e + 1] * inv);
                            w[e] = *reinterpret_cast<unsigned*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
        if (clustered) cluster_sync();             // nobody leaves while its shared memory may still be read
        if (stamp && lane == 0) {
            long long* dst = a.timing + 16ll * (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
            dst[14] = t_role - t_entry;
            dst[15] = (int)clock() - t_entry;
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            dst[6] = smid;
            dst[12] = (long long)g_entry;
            dst[13] = (long long)global_ns();
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)A_TMEM_COLS) : "memory");
    }
}

#endif  // MLC_ATTENTION_TCGEN05

}  // namespace mlc

using namespace mlc;

// q, out: bfloat16 [n_tokens][q_heads*hd], 16-byte aligned; the cache entry starts `entry_offset` elements into the
// pools and holds `pool_pages` pages of 64 tokens, [page][kv_head][64][hd].  hd is the head size the library was
// built for (64 or 128; other sizes and pages of another length are refused with MLC_ERR_UNSUPPORTED).  status: one int on the device, 0 before the call; a bounded wait that
// ran out leaves 11, 12 or 13 there.  n_splits (1, 2 or 4): that many blocks, one cluster, share out each row tile's keys
// and merge through distributed shared memory: for steps with too few row tiles to fill the GPU.  timing: null, or [blocks][16] int64 that receive the clock cycles one softmax
// warp (0-6; 7 is the block's number of tiles) and the issuing thread (8-13) of each block spent in their phases.
extern "C" int mlc_attention_tcgen05(const void* q, void* out, const int* cu_seqlens, const int* start_pos, int n_seqs,
                                     int n_tokens, int max_q_len, int q_heads, int kv_heads, int hd, float scale, int window,
                                     int n_splits, int* status, void* k_pool, void* v_pool, const int* page_table, long long entry_offset,
                                     int pages_per_seq, int page_size, long long pool_pages, long long* timing, void* stream) {
#if MLC_ATTENTION_TCGEN05
    if (hd != A_HD || page_size != A_BN) return MLC_ERR_UNSUPPORTED;
    if (n_seqs <= 0 || n_tokens <= 0 || max_q_len <= 0) return 0;
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || status == nullptr || pool_pages <= 0) return MLC_ERR_BAD_SIZE;
    if (!(scale > 0.0f) || window < 0 || n_splits < 1 || n_splits > 4) return MLC_ERR_BAD_SIZE;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || (entry_offset & 7)) return MLC_ERR_BAD_SIZE;
    const int group = q_heads / kv_heads;
    TcAttnArgs a{};
    a.out = out;
    a.cu_seqlens = cu_seqlens;
    a.start_pos = start_pos;
    a.page_table = page_table;
    a.pages_per_seq = pages_per_seq;
    a.q_heads = q_heads;
    a.kv_heads = kv_heads;
    a.group = group;
    a.heads_per_block = group < A_BM ? group : A_BM;
    a.tokens_per_block = A_BM / a.heads_per_block;
    a.head_chunks = (group + a.heads_per_block - 1) / a.heads_per_block;
    a.window = window;
    a.n_splits = n_splits;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.status = status;
    a.timing = timing;
    if (a.tokens_per_block > 256 || a.heads_per_block > 256) return MLC_ERR_BAD_SIZE;

    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)q_heads, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_heads * hd * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)a.heads_per_block, (cuuint32_t)a.tokens_per_block};
        int rc = make_tensor_map(&mq, q, 3, dims, strides, box);
        if (rc) return rc;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)pool_pages * kv_heads * A_BN};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)A_BN};
        int rc = make_tensor_map(&mk, (const bf16*)k_pool + entry_offset, 2, dims, strides, box);
        if (rc) return rc;
        rc = make_tensor_map(&mv, (const bf16*)v_pool + entry_offset, 2, dims, strides, box);
        if (rc) return rc;
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const dim3 grid(kv_heads * a.head_chunks * n_seqs * n_splits, (max_q_len + a.tokens_per_block - 1) / a.tokens_per_block, 1);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(A_THREADS);
    cfg.dynamicSmemBytes = (size_t)A_SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (n_splits > 1) {                        // blockIdx.x = (sequence, head, split): the splits of a row tile are neighbours
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = (unsigned)n_splits;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_tcgen05_kernel, mq, mk, mv, a);
    return e == cudaSuccess ? 0 : (int)e;
#else
    return MLC_ERR_UNSUPPORTED;
#endif
}

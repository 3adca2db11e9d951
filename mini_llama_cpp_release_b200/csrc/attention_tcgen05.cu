// Prompt attention on the fifth-generation tensor cores: softmax(q·kᵀ·scale)·v of many tokens over
// a paged bfloat16 cache (src/forward.cpp:585-611 and src/ops.cpp:43-70 give the arithmetic), scores and outputs accumulated in
// tensor memory, operands staged in shared memory by TMA.
//
// A block owns 128 rows of one key/value head: the group's query heads of 128 / group successive
// tokens (one row per token and head, so keys are read once for the whole group), and walks the
// keys the rows may see in tiles of 64, which is one page of the cache.  Roles:
//     warp 0     one thread issues the TMA loads: the query rows once, then a ring of K pages and a ring of V pages;
//     warp 1     allocates tensor memory; one thread issues the scores S_j = Q·K_jᵀ, some tiles ahead of the rows that
//                read them, into a ring of score buffers (buffer j mod 5 with a head size of 64, j mod 4 with 128);
//     warp 2     one thread issues O += P_j·V_j (V is the MN-major operand, read as the cache holds it);
//     warps 3-   teams of four warps, one thread per row each: three teams with a head size of 64, two with 128 (tensor
//                memory holds a team's output beside the score buffers); team t takes the tiles t, t + teams, ...
//                A thread reads its row's 64 scores from tensor memory, masks where the tile meets the diagonal, a
//                window's edge or padding rows, keeps the team's running maximum and sum in float32, and writes
//                P_j = exp2(s·scale·log2e − m) as bfloat16 back into tensor memory, over the scores it has read: the
//                product with V takes P from there, so P never crosses shared memory (whose bandwidth the operands of
//                the products and the arriving pages fill).  Each team's output accumulates in tensor memory; when a row's
//                maximum rises by more than 2^8 the row's thread rescales its lane of the output there before O_j is
//                added.  At the end the teams exchange each row's (maximum, sum) and every thread adds and stores a share
//                of the row's columns.
// A block has one tile in flight per team and the scores of those after them: a team finds its next
// scores complete when it has handed over its probabilities, and neither issuing thread waits for the other's
// products (an issue costs its thread some 60 clocks and a barrier wait twice that, whatever the product's size).
// Every barrier has one waiting thread, or a team's threads in step, and a waiter knows the phase before the one
// it waits for to be complete: a parity wait cannot tell a phase from the one two before or after it.
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
    float scale_log2;
    int* status;
    long long* timing;          // optional [blocks][16] clock cycles the first softmax warp spent in each phase (0-4), the
                                // block's tiles (7), cycles from entry to the role's start (14) and end (15); or null
};

#if MLC_ATTENTION_TCGEN05

constexpr int A_HD = MLC_HEAD_DIM;
constexpr int A_BM = 128;                              // rows of a block
constexpr int A_BN = 64;                               // keys of a tile: one page
constexpr int A_KB = A_HD / 64;                        // 64-element spans of the head size
constexpr int A_TEAMS = (A_HD == 64) ? 3 : 2;          // tiles in the rows' hands at a time
constexpr int A_AHEAD = (A_HD == 64) ? 5 : 4;          // score buffers and P buffers (rings): tiles the scores are ahead
constexpr int A_K_STAGES = 6;                          // K pages in flight
constexpr int A_V_STAGES = 4;
constexpr int A_Q_BYTES = A_KB * A_BM * 128;
constexpr int A_TILE_BYTES = A_KB * A_BN * 128;        // one K or V page of one head
constexpr int A_BAR_BYTES = 512 + A_TEAMS * 1024;      // barriers, then the teams' (maximum, sum) of every row [teams][128][2] floats
constexpr int A_THREADS = 96 + 128 * A_TEAMS;
constexpr int A_SMEM_BYTES = A_Q_BYTES + (A_K_STAGES + A_V_STAGES) * A_TILE_BYTES + A_BAR_BYTES + 1024 /* alignment slack */;
static_assert(A_SMEM_BYTES <= 227 * 1024, "shared memory of a block");
constexpr int A_TMEM_COLS = 512;                       // the score buffers of 64 columns, then every team's output of A_HD
constexpr int A_O_COL = A_AHEAD * A_BN;                // first column of the outputs
static_assert(A_O_COL + A_TEAMS * A_HD <= A_TMEM_COLS, "tensor memory of a block");
static_assert(A_HD % (16 * A_TEAMS) == 0 || A_TEAMS == 3, "how the teams share out the output's columns at the end");
constexpr int A_BLOCKS_PER_SM = 1;
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
    // ---- which rows: blocks are handed out x first, every sequence's and head's last rows (which see the most keys)
    // before anyone's earlier rows
    const int heads_y = a.kv_heads * a.head_chunks;
    const int b = blockIdx.x / heads_y;
    const int kvh = (blockIdx.x % heads_y) / a.head_chunks, chunk = blockIdx.x % a.head_chunks;
    const int tok0 = (gridDim.y - 1 - blockIdx.y) * a.tokens_per_block;

    extern __shared__ unsigned char smem_dyn[];
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    const unsigned q_base = base;
    const unsigned k_base = q_base + A_Q_BYTES;
    const unsigned v_base = k_base + A_K_STAGES * A_TILE_BYTES;
    constexpr unsigned v_off = A_Q_BYTES + A_K_STAGES * A_TILE_BYTES;
    const unsigned bar_base = v_base + A_V_STAGES * A_TILE_BYTES;
    constexpr unsigned bar_off = A_Q_BYTES + (A_K_STAGES + A_V_STAGES) * A_TILE_BYTES;
    // tile j's buffer in tensor memory, for its scores and then for its probabilities: j mod A_AHEAD
    constexpr int B_KE = A_K_STAGES, B_VF = 2 * A_K_STAGES, B_VE = B_VF + A_V_STAGES, B_SF = B_VE + A_V_STAGES;
    static_assert(B_SF + 4 * A_AHEAD + 3 <= 64, "the barriers' area");
    auto k_full = [&](int s) { return bar_base + 8u * s; };
    auto k_empty = [&](int s) { return bar_base + 8u * (B_KE + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (B_VF + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (B_VE + s); };
    auto s_full = [&](int i) { return bar_base + 8u * (B_SF + i); };                   // S_j complete
    auto p_full = [&](int i) { return bar_base + 8u * (B_SF + 2 * A_AHEAD + i); };     // P_j written, O rescaled: by the team's 128 threads
    auto o_full = [&](int i) { return bar_base + 8u * (B_SF + 3 * A_AHEAD + i); };     // the team's O += P_j V_j complete
    const unsigned q_full = bar_base + 8u * (B_SF + 4 * A_AHEAD);
    const unsigned v_last = bar_base + 8u * (B_SF + 4 * A_AHEAD + 1);                  // the block's last V tile has landed
    const unsigned tmem_slot = bar_base + 8u * (B_SF + 4 * A_AHEAD + 2);
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + bar_off + 8 * (B_SF + 4 * A_AHEAD + 2));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_K_STAGES; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
        }
        for (int s = 0; s < A_V_STAGES; ++s) {
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        for (int i = 0; i < A_AHEAD; ++i) {
            mbar_init(s_full(i), 1);
            mbar_init(p_full(i), 128);
            mbar_init(o_full(i), 1);
        }
        mbar_init(q_full, 1);
        mbar_init(v_last, 1);
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
    const int tile_begin = lo_block / A_BN;
    const int n_tiles = (n_tok > 0) ? p_last / A_BN + 1 - tile_begin : 0;
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
            // Two streams of pages, K and V, each held up only by its own ring: K_j wants the scores that read its stage
            // complete, V_j the product that read its stage.  The thread looks at both in turn and never waits on one
            // while the other could go (K runs ahead of V by the score buffers and its ring).
            int jk = 0, jv = 0;
            int page_k = __ldg(pages + tile_begin), page_v = page_k;
            unsigned long long deadline = 0;
            for (unsigned spin = 0; jk < n_tiles || jv < n_tiles; ++spin) {
                bool moved = false;
                if (jk < n_tiles && mbar_test(k_empty(jk % A_K_STAGES), ((jk / A_K_STAGES) & 1) ^ 1u)) {
                    const int s = jk % A_K_STAGES;
                    const int row = (page_k * a.kv_heads + kvh) * A_BN;       // a missing page (-1) reads as zeros
                    mbar_expect_tx(k_full(s), A_TILE_BYTES);
                    for (int kb = 0; kb < A_KB; ++kb)
                        tma_load_2d(k_base + s * A_TILE_BYTES + kb * A_BN * 128, &map_k, kb * 64, row, k_full(s));
                    if (++jk < n_tiles) page_k = __ldg(pages + tile_begin + jk);
                    moved = true;
                }
                if (jv < n_tiles && jv < jk && mbar_test(v_empty(jv % A_V_STAGES), ((jv / A_V_STAGES) & 1) ^ 1u)) {
                    const int s = jv % A_V_STAGES;
                    const int row = (page_v * a.kv_heads + kvh) * A_BN;
                    mbar_expect_tx(v_full(s), A_TILE_BYTES);
                    for (int kb = 0; kb < A_KB; ++kb)
                        tma_load_2d(v_base + s * A_TILE_BYTES + kb * A_BN * 128, &map_v, kb * 64, row, v_full(s));
                    if (++jv < n_tiles) page_v = __ldg(pages + tile_begin + jv);
                    moved = true;
                }
                if (moved) {
                    deadline = 0;
                } else if ((spin & 255u) == 255u) {
                    const unsigned long long now = global_ns();
                    if (deadline == 0) deadline = now + TC_WAIT_NS;
                    else if (now > deadline) {
                        atomicCAS(a.status, 0, 11);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- scores: S_j into buffer j mod A_AHEAD as soon as K_j has landed and the product that read the
        // buffer's last probabilities is complete; the commits hand S_j to its team and the K stage back to the loader
        if (lane == 0 && n_tiles > 0) {
            constexpr unsigned idesc_s = umma_idesc(A_BN);
            bool ok = mbar_wait_polling(q_full, 0, a.status, 12);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % A_K_STAGES, i = j % A_AHEAD;
                ok = mbar_wait_polling(k_full(s), (j / A_K_STAGES) & 1, a.status, 12);
                if (ok && j >= A_AHEAD) ok = mbar_wait_polling(o_full(i), (unsigned)(j / A_AHEAD - 1) & 1u, a.status, 12);
                if (!ok) break;
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
                tcgen05_commit(s_full(i));
                tcgen05_commit(k_empty(s));
            }
        }
    } else if (warp == 2) {
        // ---------------- outputs: the team's O += P_j V_j once V_j has landed and the team has written P_j (and rescaled
        // its output where needed); the commits tell that the tile's buffer is free for other scores and the team's O at
        // rest again, and hand the V stage back to the loader
        if (lane == 0 && n_tiles > 0) {
            constexpr unsigned idesc_o = umma_idesc(A_HD, true);
            bool ok = true;
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % A_V_STAGES, i = j % A_AHEAD;
                ok = mbar_wait_polling(v_full(s), (j / A_V_STAGES) & 1, a.status, 12);
                if (!ok) break;
                // the rows zero what lies beyond the sequence's end in the last V tile: told here that it has landed, since
                // this thread alone follows the V stages' barriers phase by phase
                if (j == n_tiles - 1 && (tile_begin + j) * A_BN + A_BN - 1 > seq_last) mbar_arrive(v_last);
                ok = mbar_wait_polling(p_full(i), (unsigned)(j / A_AHEAD) & 1u, a.status, 12);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned d = tmem_base + (unsigned)(A_O_COL + (j % A_TEAMS) * A_HD);
                const unsigned p_tmem = tmem_base + (unsigned)(i * A_BN);       // P_j: 32 columns of bfloat16 pairs
                const unsigned long long vd = umma_desc_sw128_mn(v_base + s * A_TILE_BYTES, A_BN * 128);
#pragma unroll
                for (int k = 0; k < 4; ++k)      // 16 keys a step: 8 columns of P, two 8-key groups of V
                    tcgen05_mma_f16_ts(d, p_tmem + 8u * k, vd + (unsigned long long)((2048u >> 4) * k), idesc_o, (j >= A_TEAMS || k > 0) ? 1u : 0u);
                tcgen05_commit(o_full(i));
                tcgen05_commit(v_empty(s));
            }
        }
    } else if (n_tiles > 0) {
        // ---------------- teams of four warps, one thread per row each.  Team t takes the tiles t, t + A_TEAMS, ..., with
        // its own running maximum and sum and its own output accumulator in tensor memory; the teams meet once, at the end.
        const int q4 = warp & 3;                  // the quarter of tensor memory's lanes this warp may read
        const int team = (warp - 3) >> 2;
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
#ifdef MLC_PHASE_STAMPS
        const bool stamp = a.timing != nullptr && warp == 3;      // the whole warp keeps time, so that it stays converged
#else
        constexpr bool stamp = false;                             // phase clocks are compiled in only with -DMLC_PHASE_STAMPS
#endif
        int ph[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t0 = 0, t1;        // 32-bit clocks: differences survive the wrap
#define MLC_PHASE(k) if (stamp) { t1 = (int)clock(); ph[k] += t1 - t0; t0 = t1; }
        if (stamp) t0 = (int)clock();
        const int t_role = t0;
        const unsigned o_taddr = tmem_base + lane_base + (unsigned)(A_O_COL + team * A_HD);
        int my_tiles = 0;

        for (int j = team; j < n_tiles; j += A_TEAMS, ++my_tiles) {
            const int sbuf = j % A_AHEAD;
            ok = mbar_wait(s_full(sbuf), (unsigned)(j / A_AHEAD) & 1u, a.status, 13);
            if (!ok) break;
            MLC_PHASE(0)                                   // waiting for the scores
            tcgen05_fence_after();
            const unsigned s_taddr = tmem_base + lane_base + (unsigned)(sbuf * A_BN);
            const int key0 = (tile_begin + j) * A_BN;
            // decided for the warp as a whole: lanes that went separate ways here would run everything below twice
            const bool masked = !__all_sync(0xffffffffu, key0 + A_BN - 1 <= hi && key0 >= lo);

            // the row's 64 scores, read once and kept in registers
            float sc[A_BN];
            static_assert(A_BN == 64, "one load of 64 columns");
            tmem_load64(s_taddr, sc);
            if (masked) {
#pragma unroll
                for (int c = 0; c < A_BN; ++c) {
                    const int kpos = key0 + c;
                    sc[c] = (kpos >= lo && kpos <= hi) ? sc[c] : -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains instead of one of 64 links
#pragma unroll
            for (int c = 0; c < A_BN; c += 4) {
                mx4[0] = fmaxf(mx4[0], sc[c]);
                mx4[1] = fmaxf(mx4[1], sc[c + 1]);
                mx4[2] = fmaxf(mx4[2], sc[c + 2]);
                mx4[3] = fmaxf(mx4[3], sc[c + 3]);
            }
            MLC_PHASE(1)                                   // reading them, maximum
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;   // the scale is positive
            const bool raise = mx > m + 8.0f;                         // false while nothing has been seen (-inf > -inf)
            const float m_new = raise ? mx : m;
            const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
            const float corr = raise ? fast_exp2(m - m_use) : 1.0f;   // 0 when nothing was seen before
            m = m_new;

            // probabilities, their sum, P as pairs of bfloat16 over the first half of the scores' columns
            float ls4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            unsigned pk[A_BN / 2];
#pragma unroll
            for (int c = 0; c < A_BN / 2; ++c) {
                const float p0 = fast_exp2(fmaf(sc[2 * c], a.scale_log2, -m_use));
                const float p1 = fast_exp2(fmaf(sc[2 * c + 1], a.scale_log2, -m_use));
                ls4[(2 * c) & 3] += p0;
                ls4[(2 * c + 1) & 3] += p1;
                __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);        // key 2c in the low half
                pk[c] = *reinterpret_cast<unsigned*>(&hh);
            }
            tmem_store32_words(s_taddr, pk);
            l = l * corr + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
            MLC_PHASE(2)                                   // exponentials, writing P

            if (j == n_tiles - 1 && key0 + A_BN - 1 > seq_last) {
                // the block's last tile reaches past the sequence's last key: zero those rows of V (whole 128-byte rows,
                // so the swizzle does not matter) once TMA has delivered the tile
                const int st = j % A_V_STAGES;
                ok = mbar_wait(v_last, 0, a.status, 13);
                if (!ok) break;
                const int first = max(seq_last + 1 - key0, 0), n_rows = A_BN - first;
                for (int idx = r; idx < n_rows * 8 * A_KB; idx += 128) {
                    const int kb = idx / (n_rows * 8), rem = idx % (n_rows * 8);
                    *reinterpret_cast<uint4*>(smem_generic + v_off + st * A_TILE_BYTES + kb * A_BN * 128 + (first + rem / 8) * 128 +
                                              (rem % 8) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_async_shared();
            }
            if (j >= A_TEAMS && __any_sync(0xffffffffu, raise)) {
                // Rescale this warp's rows of the team's output before P_j V_j is added to them, once the output is at
                // rest: when the team's last product is complete.
                ok = mbar_wait(o_full((j - A_TEAMS) % A_AHEAD), (unsigned)((j - A_TEAMS) / A_AHEAD) & 1u, a.status, 13);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < A_HD; c0 += 32) {
                    float v[32];
                    tmem_load32(o_taddr + (unsigned)c0, v);
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] *= corr;
                    tmem_store32(o_taddr + (unsigned)c0, v);
                }
            }
            tmem_store_wait();                             // P_j (and a rescaled output) is in tensor memory
            tcgen05_fence_before();
            mbar_arrive(p_full(sbuf));
            MLC_PHASE(3)                                   // zeroing, rescaling, hand-over
        }
        // the team's last product: the tensor cores complete products in the order of their issue, so the team's earlier
        // ones are complete with it
        if (ok && my_tiles > 0) {
            const int jl = team + A_TEAMS * (my_tiles - 1);
            ok = mbar_wait(o_full(jl % A_AHEAD), (unsigned)(jl / A_AHEAD) & 1u, a.status, 13);
        }
        MLC_PHASE(4)                                       // waiting for the last product
        if (stamp && lane == 0) {
            long long* dst = a.timing + 16ll * (blockIdx.x + gridDim.x * blockIdx.y);
            for (int k = 0; k < 7; ++k) dst[k] = ph[k];
            dst[7] = n_tiles;
        }
#undef MLC_PHASE
        // ---- the teams meet: each row's (maximum, sum) pairs cross through shared memory, then every thread takes a share
        // of the row's output columns (in runs of 16) and adds the teams' accumulators out of tensor memory
        float* ml = reinterpret_cast<float*>(smem_generic + bar_off + 512);            // [teams][128 rows][2]
        ml[(team * 128 + r) * 2] = m;
        ml[(team * 128 + r) * 2 + 1] = l;
        tcgen05_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(128 * A_TEAMS) : "memory");               // the softmax warps only
        tcgen05_fence_after();
        float f[A_TEAMS], m_all = -INFINITY, l_all = 0.0f;
#pragma unroll
        for (int u = 0; u < A_TEAMS; ++u) m_all = fmaxf(m_all, ml[(u * 128 + r) * 2]);       // -inf where a team had no tile
        const float m_ref = (m_all == -INFINITY) ? 0.0f : m_all;
#pragma unroll
        for (int u = 0; u < A_TEAMS; ++u) {
            f[u] = (n_tiles > u) ? fast_exp2(ml[(u * 128 + r) * 2] - m_ref) : 0.0f;
            l_all += (n_tiles > u) ? ml[(u * 128 + r) * 2 + 1] * f[u] : 0.0f;
        }
        const float inv = 1.0f / l_all;
        // runs of 16 columns: two teams take half of them each; three teams (64 columns) take 2, 1 and 1
        constexpr int RUNS = A_HD / 16;
        const int run0 = (A_TEAMS == 3) ? (team == 0 ? 0 : team + 1) : team * (RUNS / A_TEAMS);
        const int n_runs = (A_TEAMS == 3) ? (team == 0 ? 2 : 1) : RUNS / A_TEAMS;
        static_assert(A_TEAMS != 3 || RUNS == 4, "three teams share out four runs of columns");
        bf16* dst = (bf16*)a.out + ((long long)(seq_tok0 + tok0 + t) * a.q_heads + kvh * a.group + hg) * A_HD;
        const unsigned o_first = tmem_base + lane_base + (unsigned)A_O_COL;
        for (int run = run0; run < run0 + n_runs; ++run) {
            float acc[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) acc[c] = 0.0f;
#pragma unroll
            for (int u = 0; u < A_TEAMS; ++u) {
                if (n_tiles > u) {                         // the same for the whole block: every lane takes part in the load
                    float v[16];
                    tmem_load16(o_first + (unsigned)(u * A_HD + 16 * run), v);
#pragma unroll
                    for (int c = 0; c < 16; ++c) acc[c] = fmaf(v[c], f[u], acc[c]);
                }
            }
            if (row_ok && ok) {
                unsigned wd[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
                    wd[e] = *reinterpret_cast<unsigned*>(&hh);
                }
                *reinterpret_cast<uint4*>(dst + 16 * run) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
                *reinterpret_cast<uint4*>(dst + 16 * run + 8) = make_uint4(wd[4], wd[5], wd[6], wd[7]);
            }
        }
        if (stamp && lane == 0) {
            long long* dstt = a.timing + 16ll * (blockIdx.x + gridDim.x * blockIdx.y);
            dstt[14] = t_role - t_entry;
            dstt[15] = (int)clock() - t_entry;
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
// ran out leaves 11, 12 or 13 there.  timing: null, or [blocks][16] int64 that receive the clock cycles the first team's
// first warp of each block spent in its phases (0 waiting for scores, 1 reading them, 2 exponentials and P, 3 hand-over,
// 4 waiting for the last product), the block's number of tiles (7), and the cycles from the block's entry to that
// warp's start (14) and end (15).
extern "C" int mlc_attention_tcgen05(const void* q, void* out, const int* cu_seqlens, const int* start_pos, int n_seqs,
                                     int n_tokens, int max_q_len, int q_heads, int kv_heads, int hd, float scale, int window,
                                     int* status, void* k_pool, void* v_pool, const int* page_table, long long entry_offset,
                                     int pages_per_seq, int page_size, long long pool_pages, long long* timing, void* stream) {
#if MLC_ATTENTION_TCGEN05
    if (hd != A_HD || page_size != A_BN) return MLC_ERR_UNSUPPORTED;
    if (n_seqs <= 0 || n_tokens <= 0 || max_q_len <= 0) return 0;
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || status == nullptr || pool_pages <= 0) return MLC_ERR_BAD_SIZE;
    if (!(scale > 0.0f) || window < 0) return MLC_ERR_BAD_SIZE;
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
    const dim3 grid(kv_heads * a.head_chunks * n_seqs, (max_q_len + a.tokens_per_block - 1) / a.tokens_per_block, 1);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    cudaError_t e = launch_pdl(attention_tcgen05_kernel, grid, dim3(A_THREADS), (size_t)A_SMEM_BYTES, (cudaStream_t)stream, mq, mk, mv, a);
    return e == cudaSuccess ? 0 : (int)e;
#else
    return MLC_ERR_UNSUPPORTED;
#endif
}

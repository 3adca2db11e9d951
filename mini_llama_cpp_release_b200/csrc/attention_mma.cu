// Attention over the paged cache on the tensor cores, for bfloat16 activations and cache,
// compiled for one head size (-DMLC_HEAD_DIM=16, 32, ..., 256).
//
// The arithmetic is the reference's (score = (q·k)·1/sqrt(hd) over keys lo(p)..p, softmax,
// weighted sum of values, query head h on kv head h/(H/KV): src/forward.cpp:524-526,
// 585-611; src/ops.cpp:43-70) with the usual streaming form of the softmax: a running
// maximum and sum per row in float32, scores and accumulators in float32, probabilities
// rounded to bfloat16 only as the operand of the second product.
//
// Shape of the work.  A block has four warps and a tile of 16·RT rows; a row is one
// (token, query head) pair, and all rows of a block share one kv head, so the G query heads
// of a group ride on the same key and value tiles (for 14 heads on 2 kv heads: 9 tokens x 7
// heads per 64-row tile).  Keys come in tiles of 64, one cache page, copied to shared
// memory with cp.async, two to four tiles ahead (the single-token kernel further down: by TMA at head sizes 64 and 128).
//   RT = 4: each warp owns 16 rows and walks all 64 keys of a tile (prompts, chunks).
//   RT = 1: the block has 16 rows (one decoded token's group of heads) and the four warps
//           split each tile's keys 4 x 16, merging their partial results at the end.
//   RT = 2: 32 rows, two warps per row tile, 2 x 32 keys.
// A sequence's key range can also be split over blocks (n_splits); partial (max, sum,
// weighted values) then go to scratch memory and mlc_attention_combine merges them.
#include "tcgen05.cuh"      // mbarriers with bounded waits, TMA tile loads, tensor maps

#ifndef MLC_HEAD_DIM
#error "compile with -DMLC_HEAD_DIM=<head size>"
#endif

namespace mlc {

constexpr int HD = MLC_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be 16, 32, ..., 256");
constexpr int TILE = 64;                 // keys per tile = tokens per cache page
constexpr int STRIDE = HD + 8;           // shared-memory row stride in elements: 16 bytes of padding keep ldmatrix conflict-free
constexpr int CPR = HD / 8;              // 16-byte chunks per row
constexpr int KS_QK = HD / 16;           // k-steps of q·k
constexpr int NT_O = HD / 8;             // output n-tiles
constexpr bool Q_IN_REGS = (HD <= 128);
constexpr int NSTAGE = (HD <= 64) ? 3 : 2;   // key/value tiles in flight per block
constexpr int MAX_TILES_STAGED = 1024;   // page numbers kept in shared memory (65,536 keys); later tiles look theirs up

struct MmaArgs {
    const bf16* q;            // [N][H][HD]
    bf16* out;                // [N][H][HD]
    const int* cu_seqlens;    // [B+1]
    const int* start_pos;     // [B]
    float* part_ml;           // [N*H][n_splits][2]
    float* part_o;            // [N*H][n_splits][HD]
    float scale_log2;         // scale * log2(e)
    int q_heads;
    int group;
    int window;
    int tokens_per_block;
    int heads_per_block;
    int head_chunks;
    int n_splits;
    int one_token_each;       // decode kernel: every sequence brings exactly one token, so sequence b's token is token b
    int cluster_merge;        // decode kernel: the blocks of one row tile form a cluster and merge their key splits through
                              // distributed shared memory instead of part_ml / part_o and a second kernel
    unsigned long long* stamps;   // decode kernel: null, or [blocks][12] nanosecond stamps of each block's phases
    int* status;              // decode kernel with TMA loads: where a wait that ran out leaves its code (31)
};

__device__ __forceinline__ unsigned long long stamp_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const bf16* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_at(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans_at(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const bf16* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <int RT>
__global__ void __launch_bounds__(128)
attention_mma_kernel(MmaArgs a, PagedKV c) {
    constexpr int KP = 4 / RT;             // warps sharing a row tile, each with its part of a key tile
    constexpr int KEYS_W = TILE / KP;      // keys per warp per tile
    constexpr int NT_S = KEYS_W / 8;       // score n-tiles per warp
    constexpr int KS_PV = KEYS_W / 16;     // k-steps of p·v per warp
    constexpr int ROWS = 16 * RT;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [ROWS][STRIDE]
    bf16* Ks = Qs + ROWS * STRIDE;                                // [NSTAGE][TILE][STRIDE]
    bf16* Vs = Ks + NSTAGE * TILE * STRIDE;                       // [NSTAGE][TILE][STRIDE]

    grid_launch_dependents();
    grid_dependency_wait();                    // queries and the step's keys were written by the kernel before
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
    const int GH = a.heads_per_block;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rt = warp % RT, part = warp / RT;

    // ---- stage the query rows (zeros for rows that do not exist)
    for (int idx = tid; idx < ROWS * CPR; idx += 128) {
        const int r = idx / CPR, ch = idx % CPR;
        const int t = r / GH, hg = chunk * GH + r % GH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < n_tok && hg < a.group) {
            const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
            v = *reinterpret_cast<const uint4*>(a.q + row * HD + ch * 8);
        }
        *reinterpret_cast<uint4*>(Qs + r * STRIDE + ch * 8) = v;
    }

    // ---- key range of the block and of this split, in tiles
    const int p_first = start + tok0, p_last = start + tok0 + n_tok - 1;
    const int lo_block = (a.window > 0) ? max(0, p_first - a.window + 1) : 0;
    const int tile_begin = lo_block / TILE, tile_end = p_last / TILE + 1;
    const int per_split = (tile_end - tile_begin + a.n_splits - 1) / a.n_splits;
    const int my_begin = tile_begin + split * per_split;
    const int my_end = min(tile_end, my_begin + per_split);

    // the pages of this block's tiles, fetched once: a lookup in global memory per tile would put
    // its latency in front of every tile's copies
    __shared__ int tile_pages[MAX_TILES_STAGED];
    for (int t = my_begin + tid; t < my_end && t - my_begin < MAX_TILES_STAGED; t += 128)
        tile_pages[t - my_begin] = __ldg(c.page_table + (long long)b * c.pages_per_seq + t);
    __syncthreads();

    const bf16* kp = (const bf16*)c.k_pool;
    const bf16* vp = (const bf16*)c.v_pool;
    auto load_tile = [&](int stage, int tile) {
        const int page = (tile - my_begin < MAX_TILES_STAGED) ? tile_pages[tile - my_begin]
                                                              : __ldg(c.page_table + (long long)b * c.pages_per_seq + tile);
        const long long base = c.entry_offset + ((long long)max(page, 0) * c.kv_heads + kvh) * TILE * HD;
        bf16* kd = Ks + stage * TILE * STRIDE;
        bf16* vd = Vs + stage * TILE * STRIDE;
        for (int idx = tid; idx < TILE * CPR; idx += 128) {
            const int j = idx / CPR, ch = idx % CPR;
            const int kpos = tile * TILE + j;
            const bool valid = page >= 0 && kpos >= lo_block && kpos <= p_last;
            const long long off = valid ? base + (long long)j * HD + ch * 8 : 0;
            cp_async_16(kd + j * STRIDE + ch * 8, kp + off, valid);
            cp_async_16(vd + j * STRIDE + ch * 8, vp + off, valid);
        }
    };

    // ---- this thread's two rows (lane/4 and lane/4 + 8 of the warp's row tile)
    int row_hi[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = rt * 16 + (lane >> 2) + 8 * e;
        const int t = r / GH, hg = chunk * GH + r % GH;
        row_ok[e] = (t < n_tok) && (hg < a.group);
        row_hi[e] = row_ok[e] ? start + tok0 + t : -1;
        row_lo[e] = (a.window > 0) ? max(0, row_hi[e] - a.window + 1) : 0;
    }
    // the warp's rows span these positions (rows are ordered by token)
    const int warp_t_first = (rt * 16) / GH, warp_t_last = min((rt * 16 + 15) / GH, n_tok - 1);
    const int warp_hi = start + tok0 + warp_t_last;
    const int warp_lo = (a.window > 0) ? max(0, start + tok0 + warp_t_first - a.window + 1) : 0;
    const bool warp_has_rows = warp_t_first < n_tok;
    const int warp_first_pos = start + tok0 + warp_t_first;                       // keys up to here are visible to every row of the warp
    const int warp_lo_last = (a.window > 0) ? max(0, warp_hi - a.window + 1) : 0;   // keys from here on are inside every row's window

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    unsigned qf[Q_IN_REGS ? KS_QK : 1][4];

    // tiles my_begin .. my_begin + NSTAGE - 2 are requested before the loop; every iteration requests
    // one more and waits until all but the NSTAGE - 1 newest requests have landed
#pragma unroll
    for (int p = 0; p < NSTAGE - 1; ++p) {
        if (my_begin + p < my_end) load_tile(p, my_begin + p);
        cp_async_commit();
    }
    __syncthreads();                       // Qs is staged
    if (Q_IN_REGS) {
#pragma unroll
        for (int kk = 0; kk < KS_QK; ++kk)
            ldmatrix_x4(qf[Q_IN_REGS ? kk : 0], Qs + (rt * 16 + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);
    }

    for (int tile = my_begin, it = 0; tile < my_end; ++tile, ++it) {
        const int stage = it % NSTAGE;
        if (tile + NSTAGE - 1 < my_end) load_tile((it + NSTAGE - 1) % NSTAGE, tile + NSTAGE - 1);
        cp_async_commit();
        cp_async_wait<NSTAGE - 1>();
        __syncthreads();

        const int key0 = tile * TILE + part * KEYS_W;          // first key of this warp's part
        if (warp_has_rows && key0 <= warp_hi && key0 + KEYS_W - 1 >= warp_lo) {
            const bf16* kt = Ks + stage * TILE * STRIDE + part * KEYS_W * STRIDE;
            const bf16* vt = Vs + stage * TILE * STRIDE + part * KEYS_W * STRIDE;
            float s[NT_S][4];
#pragma unroll
            for (int j = 0; j < NT_S; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KS_QK; ++kk) {
                unsigned af[4];
                if (Q_IN_REGS) {
                    af[0] = qf[Q_IN_REGS ? kk : 0][0]; af[1] = qf[Q_IN_REGS ? kk : 0][1];
                    af[2] = qf[Q_IN_REGS ? kk : 0][2]; af[3] = qf[Q_IN_REGS ? kk : 0][3];
                } else {
                    ldmatrix_x4(af, Qs + (rt * 16 + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);
                }
#pragma unroll
                for (int jp = 0; jp < NT_S / 2; ++jp) {
                    unsigned bfr[4];
                    ldmatrix_x4(bfr, kt + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * STRIDE + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(s[2 * jp], af, bfr[0], bfr[1]);
                    mma_bf16(s[2 * jp + 1], af, bfr[2], bfr[3]);
                }
            }
            // mask (only where the tile meets the diagonal, a window's edge or the sequence's end), running maximum.
            // Scores stay unscaled; the scale rides in the exponent's multiply-add.
            float mx[2] = {-INFINITY, -INFINITY};
            const bool interior = key0 + KEYS_W - 1 <= warp_first_pos && key0 >= warp_lo_last;   // the same for the whole warp
            if (interior) {
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                    mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int kpos = key0 + 8 * j + 2 * (lane & 3) + (e & 1);
                        const int rr = e >> 1;
                        const bool in_range = kpos >= row_lo[rr] && kpos <= row_hi[rr];
                        const float v = in_range ? s[j][e] : -INFINITY;
                        s[j][e] = v;
                        mx[rr] = fmaxf(mx[rr], v);
                    }
                }
            }
            float corr[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
                const float m_new = fmaxf(m[rr], mx[rr] * a.scale_log2);     // the scale is positive: it commutes with max
                const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
                corr[rr] = exp2f(m[rr] - m_use);             // 0 when nothing was seen before
                m[rr] = m_new;
                mx[rr] = -m_use;
            }
            float ls[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < NT_S; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(fmaf(s[j][e], a.scale_log2, mx[e >> 1]));
                    s[j][e] = p;
                    ls[e >> 1] += p;
                }
            }
            l[0] = l[0] * corr[0] + ls[0];
            l[1] = l[1] * corr[1] + ls[1];
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            // o += p · v
#pragma unroll
            for (int kk = 0; kk < KS_PV; ++kk) {
                unsigned pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int jp = 0; jp < NT_O / 2; ++jp) {
                    unsigned bfr[4];
                    ldmatrix_x4_trans(bfr, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + jp * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * jp], pf, bfr[0], bfr[1]);
                    mma_bf16(o[2 * jp + 1], pf, bfr[2], bfr[3]);
                }
            }
        }
        __syncthreads();                   // all warps are done with this stage before it is refilled
    }

    // the row sums are still spread over the four lanes of a quad
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }

    constexpr float LN2 = 0.6931471805599453f;
    if (KP == 1) {
        // each warp owns its rows: write straight from registers
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            if (!row_ok[rr]) continue;
            const int r = rt * 16 + (lane >> 2) + 8 * rr;
            const int t = r / GH, hg = chunk * GH + r % GH;
            const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
            if (a.n_splits == 1) {
                const float inv = 1.0f / l[rr];
                bf16* dst = a.out + row * HD + 2 * (lane & 3);
#pragma unroll
                for (int j = 0; j < NT_O; ++j)
                    *reinterpret_cast<unsigned*>(dst + 8 * j) = pack_bf16(o[j][2 * rr] * inv, o[j][2 * rr + 1] * inv);
            } else {
                const long long pr = row * a.n_splits + split;
                if ((lane & 3) == 0) {
                    a.part_ml[pr * 2] = m[rr] * LN2;
                    a.part_ml[pr * 2 + 1] = l[rr];
                }
                float* dst = a.part_o + pr * HD + 2 * (lane & 3);
#pragma unroll
                for (int j = 0; j < NT_O; ++j) {
                    dst[8 * j] = o[j][2 * rr];
                    dst[8 * j + 1] = o[j][2 * rr + 1];
                }
            }
        }
        return;
    }

    // ---- several warps hold parts of the same rows: merge them through shared memory
    static_assert(2 * NSTAGE * TILE * STRIDE * sizeof(bf16) >= (4 * 16 * HD + 4 * 16 * 2) * sizeof(float), "merge buffer");
    float* Oc = reinterpret_cast<float*>(Ks);                       // [4 warps][16][HD]
    float* MLc = Oc + 4 * 16 * HD;                                  // [4 warps][16][2]
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r16 = (lane >> 2) + 8 * rr;
        float* dst = Oc + (warp * 16 + r16) * HD + 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            dst[8 * j] = o[j][2 * rr];
            dst[8 * j + 1] = o[j][2 * rr + 1];
        }
        if ((lane & 3) == 0) {
            MLc[(warp * 16 + r16) * 2] = m[rr];
            MLc[(warp * 16 + r16) * 2 + 1] = l[rr];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < ROWS * HD; idx += 128) {
        const int r = idx / HD, d = idx % HD;
        const int t = r / GH, hg = chunk * GH + r % GH;
        if (!(t < n_tok && hg < a.group)) continue;
        const int rtile = r / 16, r16 = r % 16;
        float M = -INFINITY;
#pragma unroll
        for (int p = 0; p < KP; ++p) M = fmaxf(M, MLc[((rtile + RT * p) * 16 + r16) * 2]);
        float L = 0.0f, acc = 0.0f;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
            const int w = rtile + RT * p;
            const float mw = MLc[(w * 16 + r16) * 2];
            if (mw != -INFINITY) {
                const float f = exp2f(mw - M);
                L += MLc[(w * 16 + r16) * 2 + 1] * f;
                acc += Oc[(w * 16 + r16) * HD + d] * f;
            }
        }
        const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
        if (a.n_splits == 1) {
            a.out[row * HD + d] = __float2bfloat16_rn(acc / L);
        } else {
            const long long pr = row * a.n_splits + split;
            a.part_o[pr * HD + d] = acc;
            if (d == 0) {
                a.part_ml[pr * 2] = M * LN2;
                a.part_ml[pr * 2 + 1] = L;
            }
        }
    }
}


// ------------------------------------------------------------------ decode: 16 rows, warp-private pipelines
// One decoded token per sequence gives a block at most 16 rows (the query heads of one kv head).
// With so few rows the work per key is small and what counts is how few instructions a key costs
// and how many bytes are in flight.  Each warp therefore runs on its own: it copies whole
// sub-tiles of DKT keys (keys and values) into its own three shared-memory stages, computes all 16
// rows against them, and never meets the other warps until the end, where the warps' partial
// results are merged.  Warp w of DNW takes sub-tiles w, w + DNW, w + 2 DNW, ... of the block's key range.
// The copies are TMA loads at head sizes 64 and 128 (below) and cp.async at the others.
constexpr int DNW = (HD <= 128) ? 8 : 4;                         // warps per block: two per scheduler hide each other's latencies
constexpr int DKT = (HD <= 64) ? 32 : 16;                        // keys per sub-tile
constexpr int D_STAGE = DKT * STRIDE;                            // elements per stage and operand
constexpr int D_NT_S = DKT / 8, D_KS_PV = DKT / 16;
constexpr int D_NSTAGE = 3;                                      // stages per warp: all filled before the loop, then two sub-tiles in flight while one is used
constexpr int D_TILES_STAGED = 512;                              // page numbers kept in shared memory (32,768 keys); later tiles look theirs up
constexpr int D_MAX_CLUSTER = 16;                                // the largest cluster there is
// Cluster merge: what the other blocks of a cluster send this one.  Its share of the 16 x HD outputs (at most a
// D_MAX_CLUSTER-th of them, rounded up, in four-float pieces) from every block, and every block's (maximum, sum) per row.
// Head sizes 64 and 128: a sub-tile's keys and values come by TMA (cp.async.bulk.tensor, one thread of the warp asks for a
// whole sub-tile, an mbarrier per warp and stage says when it has landed).  A row's 128-byte spans lie apart
// ([span][key][128 bytes]) and the 16-byte pieces of a span are swapped by the key's number modulo 8 (the 128-byte
// swizzle), which keeps ldmatrix free of bank conflicts without padding.  Other head sizes: cp.async into padded rows.
constexpr bool D_TMA = (HD == 64 || HD == 128);
constexpr int D_SPANS = HD / 64;                                 // 128-byte spans per row (TMA form)
constexpr int D_OPER_BYTES = DKT * HD * 2;                       // keys (or values) of one sub-tile, TMA form
constexpr int D_STAGE_BYTES = D_TMA ? 2 * D_OPER_BYTES : 2 * D_STAGE * (int)sizeof(bf16);
constexpr int D_KV_BYTES = DNW * D_NSTAGE * D_STAGE_BYTES;
constexpr int D_Q_BYTES = 16 * STRIDE * (int)sizeof(bf16);
constexpr int D_KV_OFF = D_TMA ? ((D_Q_BYTES + 1023) / 1024) * 1024 : D_Q_BYTES;      // swizzled tiles want 1024-byte alignment
constexpr int D_VPR = HD / 4;                                    // four-float pieces per row
constexpr int D_RECV_O_BYTES = (16 * D_VPR + D_MAX_CLUSTER) * 16;
constexpr int D_RECV_BYTES = D_RECV_O_BYTES + D_MAX_CLUSTER * 16 * 8;
constexpr int D_BAR_BYTES = DNW * D_NSTAGE * 8;                  // TMA form: an mbarrier per warp and stage
constexpr size_t D_SMEM_BYTES = (size_t)D_KV_OFF + D_KV_BYTES + D_RECV_BYTES + D_BAR_BYTES + (D_TMA ? 1024 : 0) /* alignment slack */;
static_assert(D_SMEM_BYTES + D_TILES_STAGED * 4 <= 227 * 1024, "shared memory of a block");

// Shared-memory address of the 16-byte piece `piece` of key `row` in a TMA-form operand tile.
__device__ __forceinline__ unsigned d_swizzled(unsigned oper, int row, int piece) {
    return oper + (unsigned)((piece >> 3) * (DKT * 128) + row * 128 + (((piece & 7) ^ (row & 7)) << 4));
}

__global__ void __launch_bounds__(DNW * 32)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, MmaArgs a, PagedKV c) {
    extern __shared__ __align__(16) unsigned char smem_dyn[];
    // the TMA form wants its tiles on 1024-byte boundaries of the shared address space
    unsigned char* smem_raw = D_TMA ? smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u) : smem_dyn;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][STRIDE]
    bf16* KVs = reinterpret_cast<bf16*>(smem_raw + D_KV_OFF);     // [DNW warps][D_NSTAGE][K | V]: [DKT][STRIDE], or the TMA form
    __shared__ int tile_pages[D_TILES_STAGED];
    // where the cluster's other blocks write; nothing else of this block lives here, so they may write at any time
    unsigned char* recv = smem_raw + D_KV_OFF + D_KV_BYTES;
    const unsigned bars = smem_u32(recv) + D_RECV_BYTES;          // [DNW][D_NSTAGE] mbarriers (TMA form)

    unsigned long long* const stamps = MLC_STAMPS_OR_NULL((a.stamps != nullptr && threadIdx.x == 0)
        ? a.stamps + 12ull * (blockIdx.x + gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z)) : nullptr);
    if (stamps) stamps[0] = stamp_ns();                                   // entry
    grid_launch_dependents();
    const int b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int y = blockIdx.y;
    const int split = y % a.n_splits;  y /= a.n_splits;
    const int chunk = y % a.head_chunks;  y /= a.head_chunks;
    const int kvh = y;
    const int tok0 = blockIdx.x * a.tokens_per_block;
    const int GH = a.heads_per_block;
    // What the kernel before this one writes is the step's queries and the step's own keys and values, at positions
    // from start_pos on.  The description of the step (page lists, positions, token ranges) was complete before the
    // step's first kernel, and the keys before start_pos were written by earlier steps.  So the page list, the position
    // and the first sub-tiles of older keys are asked for now, while the kernel before may still be running; only the
    // queries, and a sub-tile that holds a key of this step, wait for it.
    for (int t = tid; t < c.pages_per_seq && t < D_TILES_STAGED; t += DNW * 32)
        tile_pages[t] = __ldg(c.page_table + (long long)b * c.pages_per_seq + t);
    if (D_TMA && tid == 0) {
        for (int i = 0; i < DNW * D_NSTAGE; ++i) mbar_init(bars + 8u * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int start = a.start_pos[b];
    int seq_tok0, q_len;
    if (a.one_token_each) {
        seq_tok0 = b;
        q_len = 1;
    } else {
        seq_tok0 = a.cu_seqlens[b];
        q_len = a.cu_seqlens[b + 1] - seq_tok0;
    }
    if (tok0 >= q_len) return;
    const int n_tok = min(a.tokens_per_block, q_len - tok0);
    const int p_first = start + tok0, p_last = start + tok0 + n_tok - 1;
    const int lo_block = (a.window > 0) ? max(0, p_first - a.window + 1) : 0;
    const int tile_begin = lo_block / TILE, tile_end = p_last / TILE + 1;          // in 64-key pages
    const int per_split = (tile_end - tile_begin + a.n_splits - 1) / a.n_splits;
    const int my_begin = tile_begin + split * per_split;
    const int my_end = min(tile_end, my_begin + per_split);
    __syncthreads();                           // the page list is in shared memory
    if (stamps) stamps[2] = stamp_ns();                                   // page list and position have arrived

    constexpr int SUB = TILE / DKT;                     // sub-tiles per page
    const int st_begin = my_begin * SUB, st_end = my_end * SUB;
    const bf16* kp = (const bf16*)c.k_pool;
    const bf16* vp = (const bf16*)c.v_pool;
    bf16* my_stages = reinterpret_cast<bf16*>(reinterpret_cast<unsigned char*>(KVs) + warp * D_NSTAGE * D_STAGE_BYTES);
    const unsigned my_stages_s = smem_u32(my_stages);
    const unsigned my_bars = bars + 8u * (unsigned)(warp * D_NSTAGE);
    auto page_of = [&](int tile) {
        return (tile < D_TILES_STAGED) ? tile_pages[tile] : __ldg(c.page_table + (long long)b * c.pages_per_seq + tile);
    };
    auto load_sub = [&](int stage, int st) {
        const int tile = st / SUB;
        const int page = page_of(tile);
        if (D_TMA) {
            // one thread asks for the sub-tile's keys and values, whole: rows of the pool seen as [pages x kv heads x 64][HD].
            // Keys outside the row tile's range (beyond the sequence's end as a rule) come along and are dealt with
            // when the sub-tile is used.
            if (lane == 0) {
                const int row0 = (max(page, 0) * c.kv_heads + kvh) * TILE + (st % SUB) * DKT;
                const unsigned bar = my_bars + 8u * (unsigned)stage;
                const unsigned kd = my_stages_s + (unsigned)(stage * D_STAGE_BYTES);
                mbar_expect_tx(bar, 2 * D_OPER_BYTES);
#pragma unroll
                for (int h = 0; h < D_SPANS; ++h) {
                    tma_load_2d(kd + h * (DKT * 128), &map_k, h * 64, row0, bar);
                    tma_load_2d(kd + D_OPER_BYTES + h * (DKT * 128), &map_v, h * 64, row0, bar);
                }
            }
            return;
        }
        const long long base = c.entry_offset + (((long long)max(page, 0) * c.kv_heads + kvh) * TILE + (st % SUB) * DKT) * HD;
        bf16* kd = my_stages + stage * 2 * D_STAGE;
        bf16* vd = kd + D_STAGE;
#pragma unroll 4
        for (int idx = lane; idx < DKT * CPR; idx += 32) {
            const int j = idx / CPR, ch = idx % CPR;
            const int kpos = st * DKT + j;
            const bool valid = page >= 0 && kpos >= lo_block && kpos <= p_last;
            const long long off = valid ? base + (long long)j * HD + ch * 8 : 0;
            cp_async_16(kd + j * STRIDE + ch * 8, kp + off, valid);
            cp_async_16(vd + j * STRIDE + ch * 8, vp + off, valid);
        }
    };

    // ---- the warp's first sub-tiles, one for every stage, one copy group each and in order: those whose keys all lie
    // before the step's first position now, the others (the sequence's last sub-tile, as a rule) once the kernel before
    // is done.  With a few sub-tiles a warp (eight sequences: under three) its whole share is on its way before the wait.
    int st = st_begin + warp;
    int early = 0;
#pragma unroll
    for (int p = 0; p < D_NSTAGE; ++p) {
        const int sp = st + DNW * p;
        if (early == p && (sp >= st_end || sp * DKT + DKT - 1 < start)) {
            if (sp < st_end) load_sub(p, sp);
            if (!D_TMA) cp_async_commit();
            early = p + 1;
        }
    }
    if (stamps) stamps[8] = stamp_ns();                                   // warp 0 has asked for its first older keys

    grid_dependency_wait();                    // queries and the step's keys were written by the kernel before
    if (stamps) stamps[1] = stamp_ns();                                   // the kernels before are done
    constexpr int Q_PER_THREAD = (16 * CPR + DNW * 32 - 1) / (DNW * 32);
    uint4 qv[Q_PER_THREAD];
#pragma unroll
    for (int u = 0; u < Q_PER_THREAD; ++u) {
        const int idx = tid + u * DNW * 32;
        const int r = idx / CPR, ch = idx % CPR;
        const int t = r / GH, hg = chunk * GH + r % GH;
        qv[u] = make_uint4(0, 0, 0, 0);
        if (idx < 16 * CPR && t < n_tok && hg < a.group) {
            const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
            qv[u] = *reinterpret_cast<const uint4*>(a.q + row * HD + ch * 8);
        }
    }
#pragma unroll
    for (int p = 0; p < D_NSTAGE; ++p) {
        if (p >= early) {
            if (st + DNW * p < st_end) load_sub(p, st + DNW * p);
            if (!D_TMA) cp_async_commit();
        }
    }

#pragma unroll
    for (int u = 0; u < Q_PER_THREAD; ++u) {
        const int idx = tid + u * DNW * 32;
        if (idx < 16 * CPR) *reinterpret_cast<uint4*>(Qs + (idx / CPR) * STRIDE + (idx % CPR) * 8) = qv[u];
    }
    __syncthreads();

    int row_hi[2], row_lo[2];
    bool row_ok[2];
    int all_hi = 0x7fffffff, all_lo = 0;          // keys in [all_lo, all_hi] are visible to every existing row
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int r = (lane >> 2) + 8 * e;
        const int t = r / GH, hg = chunk * GH + r % GH;
        row_ok[e] = (t < n_tok) && (hg < a.group);
        row_hi[e] = row_ok[e] ? start + tok0 + t : -1;
        row_lo[e] = (a.window > 0) ? max(0, row_hi[e] - a.window + 1) : 0;
    }
    all_hi = start + tok0;                                                           // the first token's position
    all_lo = (a.window > 0) ? max(0, p_last - a.window + 1) : 0;                     // the last token's window start

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    unsigned qf[Q_IN_REGS ? KS_QK : 1][4];
    if (Q_IN_REGS) {
#pragma unroll
        for (int kk = 0; kk < KS_QK; ++kk)
            ldmatrix_x4(qf[Q_IN_REGS ? kk : 0], Qs + (lane & 15) * STRIDE + kk * 16 + (lane >> 4) * 8);
    }

    if (stamps) stamps[3] = stamp_ns();                                   // queries staged, first keys requested
    for (int it = 0; st < st_end; st += DNW, ++it) {
        const int stage = it % D_NSTAGE;
        if (it > 0) {
            // every stage was filled before the loop; the stage read out in the last round takes the sub-tile two on
            if (st + DNW * (D_NSTAGE - 1) < st_end) load_sub((it + D_NSTAGE - 1) % D_NSTAGE, st + DNW * (D_NSTAGE - 1));
            if (!D_TMA) cp_async_commit();
        }
        const int key0 = st * DKT;
        const unsigned kt_s = my_stages_s + (unsigned)(stage * D_STAGE_BYTES), vt_s = kt_s + D_OPER_BYTES;     // TMA form
        if (D_TMA) {
            if (!mbar_wait(my_bars + 8u * (unsigned)stage, (unsigned)(it / D_NSTAGE) & 1u, a.status, 31)) break;
            // keys outside the row tile's range, or of a page the sequence does not hold, count as zeros (their scores
            // are masked below, but a value row that is not a number would spoil 0 · v)
            const int page = page_of(st / SUB);
            if (page < 0 || key0 < lo_block || key0 + DKT - 1 > p_last) {
                for (int idx = lane; idx < DKT * CPR; idx += 32) {
                    const int j = idx / CPR, ch = idx % CPR;
                    const int kpos = key0 + j;
                    if (page < 0 || kpos < lo_block || kpos > p_last) {
                        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d_swizzled(kt_s, j, ch)), "r"(z.x), "r"(z.y), "r"(z.z), "r"(z.w) : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(d_swizzled(vt_s, j, ch)), "r"(z.x), "r"(z.y), "r"(z.z), "r"(z.w) : "memory");
                    }
                }
                fence_async_shared();              // before a later TMA load writes the stage again
            }
        } else {
            cp_async_wait<D_NSTAGE - 1>();
        }
        __syncwarp();

        if (key0 <= p_last && key0 + DKT - 1 >= lo_block) {
            const bf16* kt = my_stages + stage * 2 * D_STAGE;
            const bf16* vt = kt + D_STAGE;
            float sc[D_NT_S][4];
#pragma unroll
            for (int j = 0; j < D_NT_S; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < KS_QK; ++kk) {
                unsigned af[4];
                if (Q_IN_REGS) {
                    af[0] = qf[Q_IN_REGS ? kk : 0][0]; af[1] = qf[Q_IN_REGS ? kk : 0][1];
                    af[2] = qf[Q_IN_REGS ? kk : 0][2]; af[3] = qf[Q_IN_REGS ? kk : 0][3];
                } else {
                    ldmatrix_x4(af, Qs + (lane & 15) * STRIDE + kk * 16 + (lane >> 4) * 8);
                }
#pragma unroll
                for (int jp = 0; jp < D_NT_S / 2; ++jp) {
                    unsigned bfr[4];
                    if (D_TMA) ldmatrix_x4_at(bfr, d_swizzled(kt_s, jp * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                    else ldmatrix_x4(bfr, kt + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * STRIDE + kk * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(sc[2 * jp], af, bfr[0], bfr[1]);
                    mma_bf16(sc[2 * jp + 1], af, bfr[2], bfr[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
            const bool all_visible = key0 >= all_lo && key0 + DKT - 1 <= all_hi;       // the same for the whole warp
            if (all_visible) {
#pragma unroll
                for (int j = 0; j < D_NT_S; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = row_ok[e >> 1] ? sc[j][e] * a.scale_log2 : -INFINITY;
                        sc[j][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < D_NT_S; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int kpos = key0 + 8 * j + 2 * (lane & 3) + (e & 1);
                        const int rr = e >> 1;
                        const bool in_range = kpos >= row_lo[rr] && kpos <= row_hi[rr];
                        const float v = in_range ? sc[j][e] * a.scale_log2 : -INFINITY;
                        sc[j][e] = v;
                        mx[rr] = fmaxf(mx[rr], v);
                    }
                }
            }
            float corr[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
                mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
                const float m_new = fmaxf(m[rr], mx[rr]);
                const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
                corr[rr] = exp2f(m[rr] - m_use);
                m[rr] = m_new;
                mx[rr] = m_use;
            }
            float ls[2] = {0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < D_NT_S; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = exp2f(sc[j][e] - mx[e >> 1]);
                    sc[j][e] = p;
                    ls[e >> 1] += p;
                }
            }
            l[0] = l[0] * corr[0] + ls[0];
            l[1] = l[1] * corr[1] + ls[1];
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < D_KS_PV; ++kk) {
                unsigned pf[4];
                pf[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                pf[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                pf[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                pf[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                for (int jp = 0; jp < NT_O / 2; ++jp) {
                    unsigned bfr[4];
                    if (D_TMA) ldmatrix_x4_trans_at(bfr, d_swizzled(vt_s, kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 2 + (lane >> 4)));
                    else ldmatrix_x4_trans(bfr, vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + jp * 16 + (lane >> 4) * 8);
                    mma_bf16(o[2 * jp], pf, bfr[0], bfr[1]);
                    mma_bf16(o[2 * jp + 1], pf, bfr[2], bfr[3]);
                }
            }
        }
        __syncwarp();                      // the stage is read out before the next copy into it is issued
    }
    if (!D_TMA) cp_async_wait<0>();
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
        l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }

    // ---- merge the warps' partial results
    if (stamps) stamps[4] = stamp_ns();                                   // warp 0 is through its keys
    __syncthreads();
    if (stamps) stamps[5] = stamp_ns();                                   // every warp is
    constexpr int OS = HD + 8;                                      // row stride of the warps' outputs: a warp's eight rows
                                                                    // land on different banks (rows of HD floats would all
                                                                    // start on the same one)
    float* Oc = reinterpret_cast<float*>(KVs);                      // [DNW warps][16][OS]
    float* MLc = Oc + DNW * 16 * OS;                                // [DNW warps][16][2]
    static_assert(D_KV_BYTES >= (DNW * 16 * OS + DNW * 16 * 2 + 32 + DNW * 16) * sizeof(float), "merge buffer");
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int r16 = (lane >> 2) + 8 * rr;
        float* dst = Oc + (warp * 16 + r16) * OS + 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < NT_O; ++j) *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[j][2 * rr], o[j][2 * rr + 1]);
        if ((lane & 3) == 0) {
            MLc[(warp * 16 + r16) * 2] = m[rr];
            MLc[(warp * 16 + r16) * 2 + 1] = l[rr];
        }
    }
    __syncthreads();
    if (stamps) stamps[10] = stamp_ns();                                  // the warps' results are in shared memory
    constexpr float LN2 = 0.6931471805599453f;
    float* PMLc = MLc + DNW * 16 * 2;                               // [16][2] the block's maximum and sum per row
    float* Fc = PMLc + 32;                                          // [DNW][16] what a warp's sum and output are scaled by
    // a thread per (warp, row): the row's maximum over the warps and that warp's factor against it
    if (tid < DNW * 16) {
        const int w = tid / 16, r = tid % 16;
        float M = -INFINITY;
#pragma unroll
        for (int u = 0; u < DNW; ++u) M = fmaxf(M, MLc[(u * 16 + r) * 2]);
        const float mw = MLc[(w * 16 + r) * 2];
        Fc[w * 16 + r] = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
        if (w == 0) PMLc[2 * r] = M;
    }
    __syncthreads();
    // Cluster merge: the n_splits blocks of this row tile are one cluster (rank = split).  Block k owns the pieces
    // k * per .. (k + 1) * per - 1 of the 16 x HD outputs; every block sends each owner its partial result for the
    // owner's pieces and its (maximum, sum) of every row, straight into the owner's shared memory.  Stores to another
    // block's shared memory need no answer, so their way through the cluster overlaps the barrier that follows.
    const int S = a.n_splits;
    const int per = (16 * D_VPR + S - 1) / S;
    const unsigned recv_local = (unsigned)__cvta_generic_to_shared(recv);
    // a thread per four neighbouring outputs of a row
    for (int v = tid; v < 16 * D_VPR; v += DNW * 32) {
        const int r = v / D_VPR, d = (v % D_VPR) * 4;
        const int t = r / GH, hg = chunk * GH + r % GH;
        if (!(t < n_tok && hg < a.group) && !a.cluster_merge) continue;
        float L = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int w = 0; w < DNW; ++w) {
            const float f = Fc[w * 16 + r];
            const float4 x = *reinterpret_cast<const float4*>(Oc + (w * 16 + r) * OS + d);
            L = fmaf(MLc[(w * 16 + r) * 2 + 1], f, L);
            acc.x = fmaf(x.x, f, acc.x); acc.y = fmaf(x.y, f, acc.y); acc.z = fmaf(x.z, f, acc.z); acc.w = fmaf(x.w, f, acc.w);
        }
        const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
        if (a.cluster_merge) {
            const int owner = v / per;
            unsigned dst;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(recv_local + 16u * (unsigned)(split * per + (v - owner * per))), "r"(owner));
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
            if (d == 0) {
                const float M = PMLc[2 * r];
                for (int k = 0; k < S; ++k) {
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(recv_local + (unsigned)D_RECV_O_BYTES + 8u * (unsigned)(split * 16 + r)), "r"(k));
                    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(dst), "f"(M), "f"(L) : "memory");
                }
            }
        } else if (a.n_splits == 1) {
            const float inv = 1.0f / L;
            *reinterpret_cast<uint2*>(a.out + row * HD + d) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        } else {
            const long long pr = row * a.n_splits + split;
            a.part_o[pr * HD + d] = acc.x; a.part_o[pr * HD + d + 1] = acc.y;
            a.part_o[pr * HD + d + 2] = acc.z; a.part_o[pr * HD + d + 3] = acc.w;
            if (d == 0) {
                a.part_ml[pr * 2] = PMLc[2 * r] * LN2;
                a.part_ml[pr * 2 + 1] = L;
            }
        }
    }
    if (stamps) stamps[9] = stamp_ns();                                   // the block's warps are merged
    if (a.cluster_merge) {
        // release: this block's stores into the others' shared memory; acquire: theirs into this block's
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (stamps) stamps[6] = stamp_ns();                               // every block of the cluster has sent its results
        const float4* ro = reinterpret_cast<const float4*>(recv);                      // [S][per]
        const float2* rml = reinterpret_cast<const float2*>(recv + D_RECV_O_BYTES);    // [S][16]
        for (int i = tid; i < per; i += DNW * 32) {
            const int v = split * per + i;
            if (v >= 16 * D_VPR) break;
            const int r = v / D_VPR, d = (v % D_VPR) * 4;
            const int t = r / GH, hg = chunk * GH + r % GH;
            if (!(t < n_tok && hg < a.group)) continue;
            float M = -INFINITY, L = 0.0f;
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int k = 0; k < S; ++k) M = fmaxf(M, rml[k * 16 + r].x);
            for (int k = 0; k < S; ++k) {
                const float2 ml = rml[k * 16 + r];
                if (ml.x != -INFINITY) {
                    const float f = exp2f(ml.x - M);
                    const float4 x = ro[k * per + i];
                    L = fmaf(ml.y, f, L);
                    acc.x = fmaf(x.x, f, acc.x); acc.y = fmaf(x.y, f, acc.y); acc.z = fmaf(x.z, f, acc.z); acc.w = fmaf(x.w, f, acc.w);
                }
            }
            const long long row = (long long)(seq_tok0 + tok0 + t) * a.q_heads + (kvh * a.group + hg);
            const float inv = 1.0f / L;
            *reinterpret_cast<uint2*>(a.out + row * HD + d) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
        }
        // Nobody reads another block's shared memory after the barrier, and nobody writes it: a block may leave when it
        // has stored its share.
    }
    if (stamps) stamps[7] = stamp_ns();                                   // done
}

// How many clusters of `size` blocks of the decode kernel the GPU can hold at once (0: that size cannot be launched).
// 8 is the portable limit; 16 needs the opt-in and enough SMs per GPC.
static int decode_clusters_resident(int size) {
    static int cached[17] = {0};
    static bool known[17] = {false};
    if (size < 1 || size > 16) return 0;
    if (!known[size]) {
        const size_t smem = D_SMEM_BYTES;
        int n = 0;
        bool can = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        if (can && size > 8)
            can = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        if (can) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, (unsigned)size, 1);
            cfg.blockDim = dim3(DNW * 32);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = (unsigned)size;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, attention_decode_kernel, &cfg) != cudaSuccess) n = 0;
        }
        (void)cudaGetLastError();
        cached[size] = n;
        known[size] = true;
    }
    return cached[size];
}

static int launch_decode(const MmaArgs& a, const PagedKV& c, int pool_pages, dim3 grid, cudaStream_t s) {
    const size_t smem = D_SMEM_BYTES;
    // the cache entry's keys and values as matrices [pages x kv heads x 64 keys][HD], read in boxes of DKT keys x 64 columns
    CUtensorMap map_k, map_v;
    if (D_TMA) {
        if (pool_pages < 1 || a.status == nullptr) return MLC_ERR_BAD_SIZE;
        const long long rows = (long long)pool_pages * c.kv_heads * TILE;
        int rc = cached_map_2d(&map_k, (const bf16*)c.k_pool + c.entry_offset, rows, HD, 64, DKT);
        if (rc) return rc;
        rc = cached_map_2d(&map_v, (const bf16*)c.v_pool + c.entry_offset, rows, HD, 64, DKT);
        if (rc) return rc;
    } else {
        memset(&map_k, 0, sizeof(map_k));
        memset(&map_v, 0, sizeof(map_v));
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (!a.cluster_merge) {
        cudaError_t e = launch_pdl(attention_decode_kernel, grid, dim3(DNW * 32), smem, s, map_k, map_v, a, c);
        return e == cudaSuccess ? 0 : (int)e;
    }
    if (decode_clusters_resident(a.n_splits) < 1) return MLC_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DNW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;       // blockIdx.y = (head, split): the splits of a head are neighbours
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)a.n_splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel, map_k, map_v, a, c);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int RT>
static int launch_mma(const MmaArgs& a, const PagedKV& c, dim3 grid, cudaStream_t s) {
    constexpr int ROWS = 16 * RT;
    const size_t smem = (size_t)(ROWS + 2 * NSTAGE * TILE) * STRIDE * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = launch_pdl(attention_mma_kernel<RT>, grid, dim3(128), smem, s, a, c);
    return e == cudaSuccess ? 0 : (int)e;
}

}  // namespace mlc

using namespace mlc;

extern "C" int mlc_attention_mma_head_dim() { return HD; }

// How many clusters of `size` blocks of the single-token kernel fit on the GPU at once; 0 if clusters of that size
// cannot be launched.  Key splits merged inside a cluster (n_splits > 1 without part_ml / part_o) need at least 1.
extern "C" int mlc_attention_decode_clusters_resident(int size) { return decode_clusters_resident(size); }

// Measurement hook, effective only in builds with -DMLC_PHASE_STAMPS: later launches of the decode kernel leave
// nanosecond stamps of their phases in p ([blocks][12] on the device; null switches it off again).
extern "C" int mlc_phase_stamps_built() {
#ifdef MLC_PHASE_STAMPS
    return 1;
#else
    return 0;
#endif
}
static unsigned long long* g_decode_stamps = nullptr;
extern "C" int mlc_attention_decode_stamps(unsigned long long* p) {
    g_decode_stamps = p;
    return 0;
}

// q, out: bfloat16 [n_tokens][q_heads][HD]; the cache pools hold bfloat16 in pages of 64 tokens.
// row_tiles: 1, 2 or 4 (16, 32 or 64 rows per block); with row_tiles 1, warp_private != 0 picks the
// kernel whose warps each stream their own sub-tiles (the decode form; at head sizes 64 and 128 by TMA, for which it
// needs pool_pages, the pages of a cache entry, and status, one int on the device that is 0 before the call and holds
// 31 afterwards if a bounded wait for a sub-tile ran out).  n_splits > 1 writes partial results to
// part_ml / part_o (sizes as for mlc_attention_simt) and leaves `out` to the combine kernel.
extern "C" int mlc_attention_mma(const void* q, void* out, const int* cu_seqlens, const int* start_pos, int n_seqs,
                                 int n_tokens, int max_q_len, int q_heads, int kv_heads, int hd, float scale,
                                 int window, int row_tiles, int warp_private, int n_splits, float* part_ml, float* part_o,
                                 void* k_pool, void* v_pool, const int* page_table, long long entry_offset,
                                 int pages_per_seq, int page_size, int pool_pages, int* status, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (hd != HD || page_size != TILE) return MLC_ERR_BAD_SIZE;
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    if (row_tiles != 1 && row_tiles != 2 && row_tiles != 4) return MLC_ERR_BAD_SIZE;
    if (!(scale > 0.0f)) return MLC_ERR_BAD_SIZE;                     // the kernels move the scale past a maximum
    // key splits without partial-result buffers: the decode kernel merges them inside a cluster (up to
    // mlc_attention_decode_cluster_limit() splits)
    const bool cluster_merge = n_splits > 1 && part_ml == nullptr && part_o == nullptr;
    if (n_splits < 1 || (n_splits > 1 && !cluster_merge && (part_ml == nullptr || part_o == nullptr))) return MLC_ERR_BAD_SIZE;
    if (cluster_merge && !(row_tiles == 1 && warp_private && max_q_len == 1)) return MLC_ERR_UNSUPPORTED;
    MmaArgs a;
    a.q = (const bf16*)q;
    a.out = (bf16*)out;
    a.cu_seqlens = cu_seqlens;
    a.start_pos = start_pos;
    a.part_ml = part_ml;
    a.part_o = part_o;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.q_heads = q_heads;
    a.group = q_heads / kv_heads;
    a.window = window;
    const int rows = 16 * row_tiles;
    a.heads_per_block = a.group < rows ? a.group : rows;
    a.tokens_per_block = rows / a.heads_per_block;
    a.head_chunks = (a.group + a.heads_per_block - 1) / a.heads_per_block;
    a.n_splits = n_splits;
    a.cluster_merge = cluster_merge ? 1 : 0;
    a.one_token_each = (max_q_len == 1 && n_tokens == n_seqs) ? 1 : 0;
    a.stamps = g_decode_stamps;
    a.status = status;
    const long long gy = (long long)kv_heads * a.head_chunks * n_splits;
    if (gy > 65535) return MLC_ERR_BAD_SIZE;
    PagedKV c{k_pool, v_pool, page_table, entry_offset, pages_per_seq, page_size, kv_heads, hd};
    dim3 grid((max_q_len + a.tokens_per_block - 1) / a.tokens_per_block, (unsigned)gy, n_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    if (row_tiles == 4) return launch_mma<4>(a, c, grid, s);
    if (row_tiles == 2) return launch_mma<2>(a, c, grid, s);
    if (warp_private) return launch_decode(a, c, pool_pages, grid, s);
    return launch_mma<1>(a, c, grid, s);
}

// y[token][row] = sum_k W[row][k] · h[token][k] on the fifth-generation tensor cores:
// bfloat16 operands staged in shared memory by TMA, float32 accumulators in tensor memory,
// epilogues that finish the layer's arithmetic before anything is written.
//
// The weight matrix is the M operand: a block owns 128 rows of W (UMMA M = 128) and BN
// tokens (UMMA N = 16 ... 256), so the same kernel streams weights once for a handful of
// decoded tokens and tiles a prompt of thousands.  K runs in steps of 64 elements (one
// 128-byte swizzle span per row) through a ring of shared-memory stages:
//     warp 0   one thread issues the TMA loads of the W tile and the activation tile;
//     warp 1   allocates tensor memory, one thread issues tcgen05.mma and commits;
//     warps 2-5  read the accumulators with tcgen05.ld (each warp its 32 lanes) and run the epilogue.
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
// Every wait on an mbarrier is bounded by a clock; a wait that runs out records a code in
// `status`, the block skips its stores, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace mlc {

constexpr int G_BM = 128;
constexpr int G_BK = 64;
constexpr int G_THREADS = 192;
constexpr int G_A_BYTES = G_BM * G_BK * 2;                 // 16 KiB per stage
constexpr unsigned long long G_WAIT_NS = 2000000000ull;     // two seconds

enum { EPI_STORE = 0, EPI_SILU_MUL = 1, EPI_QKV = 2 };

struct GemmArgs {
    void* out;                 // STORE / SILU_MUL: [splits][tokens][n_out or n_out/2]; QKV: q [tokens][q_heads*hd]
    int out_dtype;
    int n_out;                 // rows of W
    int n_tok;
    int k_blocks;              // ceil(K / 64)
    int k_blocks_per_split;
    long long split_stride;    // elements between the output slices of two splits
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

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait for the phase with the given parity; false (and a code in *status) if two seconds pass.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
    unsigned long long deadline = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 1023u) == 1023u) {
            const unsigned long long now = global_ns();
            if (deadline == 0) deadline = now + G_WAIT_NS;
            else if (now > deadline) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int c0, int c1, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                                unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_load16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, swizzled in
// 128-byte spans: start address, 1024 bytes between groups of eight rows, descriptor version 1.
__device__ __forceinline__ unsigned long long umma_desc_sw128(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);            // bits 0-13: address / 16
    d |= (unsigned long long)(1024u >> 4) << 32;                       // bits 32-45: stride between 8-row groups / 16
    d |= 1ull << 46;                                                   // bits 46-47: version
    d |= 2ull << 61;                                                   // bits 61-63: 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = BN.
__host__ __device__ constexpr unsigned umma_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(bn >> 3) << 17) | ((unsigned)(G_BM >> 4) << 24);
}

template <int BN> struct GemmShape {
    static constexpr int B_BYTES = BN * G_BK * 2;
    static constexpr int STAGE_BYTES = G_A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN <= 64) ? 8 : (BN <= 128 ? 6 : 4);
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int META_BYTES = BN * 16;      // per token: position, cache offset (QKV epilogue)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + META_BYTES;
};

template <typename T> __device__ __forceinline__ void store_out(void* base, long long idx, float v) {
    ((T*)base)[idx] = from_float<T>(v);
}

template <int BN, int EPI>
__global__ void __launch_bounds__(G_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmArgs g) {
    using S = GemmShape<BN>;
    extern __shared__ unsigned char smem_dyn[];
    const unsigned base = (smem_u32(smem_dyn) + 1023u) & ~1023u;          // tiles want 1024-byte alignment
    const unsigned a_base = base;
    const unsigned b_base = base + S::STAGES * G_A_BYTES;
    const unsigned bar_base = base + S::STAGES * S::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (S::STAGES + s); };
    const unsigned accum_bar = bar_base + 8u * (2 * S::STAGES);
    const unsigned tmem_slot = bar_base + 8u * (2 * S::STAGES + 1);
    unsigned char* smem_generic = smem_dyn + (base - smem_u32(smem_dyn));
    volatile unsigned* tmem_slot_ptr = reinterpret_cast<volatile unsigned*>(smem_generic + S::STAGES * S::STAGE_BYTES + 8 * (2 * S::STAGES + 1));
    int* tok_pos = reinterpret_cast<int*>(smem_generic + S::STAGES * S::STAGE_BYTES + 256);              // [BN]
    long long* tok_off = reinterpret_cast<long long*>(tok_pos + BN);                                      // [BN], 8-byte aligned: BN*4 is a multiple of 8

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * G_BM, n0 = blockIdx.y * BN, split = blockIdx.z;
    const int kb_begin = split * g.k_blocks_per_split;
    const int kb_end = min(g.k_blocks, kb_begin + g.k_blocks_per_split);
    const int n_kb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S::STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((unsigned)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const unsigned tmem_acc = *tmem_slot_ptr;

    grid_launch_dependents();                  // the next kernel may start its own set-up now
    if (warp == 0) {
        // ---------------- TMA producer.  The weights do not depend on the kernels before this one: the first
        // round of weight tiles is requested before the wait for those kernels, the activations after it.
        if (lane == 0) {
            const int early = min(n_kb, S::STAGES);
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                tma_load_2d(a_base + i * G_A_BYTES, &map_w, (kb_begin + i) * G_BK, m0, full_bar(i));
            }
            grid_dependency_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(b_base + i * S::B_BYTES, &map_x, (kb_begin + i) * G_BK, n0, full_bar(i));
            for (int i = early; i < n_kb; ++i) {
                const int s = i % S::STAGES;
                const unsigned phase = (i / S::STAGES) & 1;
                if (!mbar_wait(empty_bar(s), phase ^ 1u, g.status, 1)) break;
                mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                const int k = (kb_begin + i) * G_BK;
                tma_load_2d(a_base + s * G_A_BYTES, &map_w, k, m0, full_bar(s));
                tma_load_2d(b_base + s * S::B_BYTES, &map_x, k, n0, full_bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc = umma_idesc(BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % S::STAGES;
                const unsigned phase = (i / S::STAGES) & 1;
                ok = mbar_wait(full_bar(s), phase, g.status, 2);
                if (!ok) break;
                tcgen05_fence_after();
                const unsigned long long a_desc = umma_desc_sw128(a_base + s * G_A_BYTES);
                const unsigned long long b_desc = umma_desc_sw128(b_base + s * S::B_BYTES);
#pragma unroll
                for (int k = 0; k < G_BK / 16; ++k) {
                    // 16 elements = 32 bytes further along K inside the swizzle span: +2 in address/16 units
                    tcgen05_mma_f16(tmem_acc, a_desc + 2ull * k, b_desc + 2ull * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(empty_bar(s));          // the stage is free once these products have read it
            }
            tcgen05_commit(accum_bar);                 // arrives when every product issued so far is done
        }
    } else {
        // ---------------- epilogue: warp q reads tensor-memory lanes 32q .. 32q+31
        const int q = warp & 3;
        grid_dependency_wait();                // positions, page lists and the output buffers may come from earlier kernels
        if (EPI == EPI_QKV) {
            for (int t = threadIdx.x - 64; t < BN; t += 128) {
                int p = 0;
                long long off = 0;
                if (n0 + t < g.n_tok) {
                    p = __ldg(g.positions + n0 + t);
                    if (g.kv_heads > 0) off = paged_offset(g.cache, __ldg(g.tok_seq + n0 + t), p, 0);
                }
                tok_pos[t] = p;
                tok_off[t] = off;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps only
        }
        const bool ok = mbar_wait(accum_bar, 0, g.status, 3);
        tcgen05_fence_after();
        const int row = m0 + q * 32 + lane;
        if (ok && n_kb > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                tmem_load16(tmem_acc + ((unsigned)(q * 32) << 16) + (unsigned)c0, v);
                if (EPI == EPI_STORE) {
                    if (row < g.n_out) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = n0 + c0 + j;
                            if (tok < g.n_tok) {
                                const long long idx = (long long)split * g.split_stride + (long long)tok * g.n_out + row;
                                if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, v[j]);
                                else store_out<bf16>(g.out, idx, v[j]);
                            }
                        }
                    }
                } else if (EPI == EPI_SILU_MUL) {
                    // even lane: gate_j, odd lane: up_j, j = row / 2
                    const int half_out = g.n_out >> 1;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                        const int tok = n0 + c0 + j;
                        if ((lane & 1) == 0 && row < g.n_out && tok < g.n_tok) {
                            const float gate = v[j], up = other;
                            const float act = gate * (1.0f / (1.0f + expf(-gate))) * up;
                            const long long idx = (long long)tok * half_out + (row >> 1);
                            if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, act);
                            else store_out<bf16>(g.out, idx, act);
                        }
                    }
                } else {
                    // QKV: stored row order inside a head is (0, hd/2, 1, hd/2+1, ...): even lane holds
                    // dim i = (row % hd) / 2, its odd neighbour dim i + hd/2.  Positions and cache offsets
                    // of the tile's tokens were put in shared memory while the products ran.
                    const int hd = g.hd, half = hd >> 1;
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
                    for (int j = 0; j < 16; ++j) {
                        const int t = c0 + j;
                        cs[j] = make_float2(1.0f, 0.0f);
                        if (rotate && row_ok && n0 + t < g.n_tok)
                            cs[j] = __ldg(g.rope + (long long)min(tok_pos[t], g.rope_positions - 1) * half + i);
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = c0 + j;
                        const float mine = v[j] + b;
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        // first half: x0·c − x1·s; second half: x0·s + x1·c, with (x0, x1) = (dim i, dim i + hd/2)
                        const float y = second ? (other * cs[j].y + mine * cs[j].x) : (mine * cs[j].x - other * cs[j].y);
                        if (!row_ok || n0 + t >= g.n_tok) continue;
                        if (is_q) {
                            const long long idx = ((long long)(n0 + t) * g.q_heads + head) * hd + d;
                            if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(g.out, idx, y);
                            else store_out<bf16>(g.out, idx, y);
                        } else {
                            void* pool = is_k ? g.cache.k_pool : g.cache.v_pool;
                            const long long off = tok_off[t] + head_off;
                            if (g.out_dtype == MLC_DTYPE_F32) store_out<float>(pool, off, y);
                            else store_out<bf16>(pool, off, y);
                        }
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"((unsigned)S::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled encode_tiled() {
    static PFN_cuTensorMapEncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (PFN_cuTensorMapEncodeTiled)p;
    }
    return fn;
}

// A row-major bfloat16 matrix [rows][cols] read in boxes of box_rows x 64 columns with the 128-byte swizzle;
// reads outside the matrix give zeros.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    PFN_cuTensorMapEncodeTiled fn = encode_tiled();
    if (fn == nullptr) return MLC_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)G_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MLC_ERR_BAD_SIZE;
}

template <int BN, int EPI>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, dim3 grid, cudaStream_t s) {
    using S = GemmShape<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = launch_pdl(gemm_tcgen05_kernel<BN, EPI>, grid, dim3(G_THREADS), (size_t)S::SMEM_BYTES, s, mw, mx, g);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int EPI>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& g, dim3 grid, cudaStream_t s) {
    switch (bn) {
        case 16: return launch_gemm<16, EPI>(mw, mx, g, grid, s);
        case 32: return launch_gemm<32, EPI>(mw, mx, g, grid, s);
        case 64: return launch_gemm<64, EPI>(mw, mx, g, grid, s);
        case 128: return launch_gemm<128, EPI>(mw, mx, g, grid, s);
        case 256: return launch_gemm<256, EPI>(mw, mx, g, grid, s);
    }
    return MLC_ERR_BAD_SIZE;
}

}  // namespace mlc

using namespace mlc;

// x: bfloat16 [n_tok][K]; w: bfloat16 [n_out][K] (K a multiple of 8, both 16-byte aligned).
// epilogue 0: out [n_splits][n_tok][n_out] (float32 or bfloat16): with n_splits > 1 the K range is shared out over
// blocks and each leaves its partial sums in its own slice for the consumer to add; 1: out [n_tok][n_out/2],
// n_splits must be 1;
// 2: out = q [n_tok][q_heads*hd], k and v go to the cache, n_splits must be 1.
// block_tokens: 16, 32, 64, 128 or 256.  status: one int on the device, 0 before the call; a bounded
// wait that ran out leaves 1 (loader), 2 (tensor cores) or 3 (epilogue) there.
extern "C" int mlc_gemm_tcgen05(const void* x, const void* w, void* out, int out_dtype, int n_tok, int n_out, int K,
                                int block_tokens, int n_splits, int epilogue, int* status, const float* bias,
                                const int* positions, const int* tok_seq, const void* rope_table, int rope_positions,
                                int q_heads, int kv_heads, int hd, void* k_pool, void* v_pool, const int* page_table,
                                long long entry_offset, int pages_per_seq, int page_size, void* stream) {
    if (n_tok <= 0 || n_out <= 0) return 0;
    if (K <= 0 || (K & 7) || (((uintptr_t)x | (uintptr_t)w) & 15)) return MLC_ERR_BAD_SIZE;
    if (out_dtype != MLC_DTYPE_F32 && out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    if (n_splits < 1 || (epilogue != EPI_STORE && n_splits != 1) || status == nullptr) return MLC_ERR_BAD_SIZE;
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
    dim3 grid((n_out + G_BM - 1) / G_BM, (n_tok + block_tokens - 1) / block_tokens, n_splits);
    if (grid.y > 65535 || grid.z > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (epilogue == EPI_STORE) return dispatch_bn<EPI_STORE>(block_tokens, mw, mx, g, grid, s);
    if (epilogue == EPI_SILU_MUL) return dispatch_bn<EPI_SILU_MUL>(block_tokens, mw, mx, g, grid, s);
    if (epilogue == EPI_QKV) return dispatch_bn<EPI_QKV>(block_tokens, mw, mx, g, grid, s);
    return MLC_ERR_UNSUPPORTED;
}

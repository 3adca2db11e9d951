// Inline-PTX wrappers for the fifth-generation tensor cores of sm_100a: mbarriers with bounded
// waits, TMA tile loads, tcgen05.mma with shared-memory operand descriptors, tensor-memory loads.
// Shared by the matrix-product kernel and the prompt attention kernel.
#pragma once

#include "common.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

#include <functional>
#include <mutex>
#include <unordered_map>

namespace mlc {

constexpr unsigned long long TC_WAIT_NS = 2000000000ull;     // a wait on a barrier gives up after two seconds

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
// Wait for the phase with the given parity; false (and a code in *status) if two seconds pass.  try_wait lets
// the hardware suspend the thread for a while instead of spinning through the issue slots other warps need.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int* status, int code) {
    unsigned long long deadline = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 63u) == 63u) {
            // a wait that another thread, block or earlier kernel already gave up: what this one waits for will not
            // come either, and a chain of kernels must not spend the full time in each of its waits
            if (spin > 4096u && *reinterpret_cast<volatile int*>(status) != 0) return false;
            const unsigned long long now = global_ns();
            if (deadline == 0) deadline = now + TC_WAIT_NS;
            else if (now > deadline) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
// One look at a barrier: whether the phase with the given parity is complete.
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// The same for a thread whose wake-up is on everyone's critical path (one that issues tensor-core work): test_wait
// polls and never suspends the thread.
__device__ __forceinline__ bool mbar_wait_polling(unsigned bar, unsigned parity, int* status, int code) {
    unsigned long long deadline = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 1023u) == 1023u) {
            if (spin > 65536u && *reinterpret_cast<volatile int*>(status) != 0) return false;
            const unsigned long long now = global_ns();
            if (deadline == 0) deadline = now + TC_WAIT_NS;
            else if (now > deadline) {
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
// mbar_wait for a barrier that threads of other blocks of the cluster arrive on: the wait acquires at cluster scope.
__device__ __forceinline__ bool mbar_wait_cluster(unsigned bar, unsigned parity, int* status, int code) {
    unsigned long long deadline = 0;
    for (unsigned spin = 0;; ++spin) {
        unsigned ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 1023u) == 1023u) {
            if (spin > 65536u && *reinterpret_cast<volatile int*>(status) != 0) return false;
            const unsigned long long now = global_ns();
            if (deadline == 0) deadline = now + TC_WAIT_NS;
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

// Instruction descriptor: bfloat16 x bfloat16 -> float32, A K-major, M = 128, N = n; B is K-major
// ([n][k], k contiguous) or, with b_mn_major, MN-major ([k][n], n contiguous).
__host__ __device__ constexpr unsigned umma_idesc(int n, bool b_mn_major = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(128 >> 4) << 24);
}

// This block's shared-memory address `addr` as an address in the shared memory of block `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_map(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Arrive on an mbarrier of another block of the cluster (address from cluster_map); this thread's earlier writes to
// that block's shared memory are visible to whoever acquires the barrier's phase.
__device__ __forceinline__ void mbar_arrive_remote(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// All threads of all blocks of the cluster meet (every thread of a warp together).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap* map, int c0, int c1, int c2, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
// Makes this thread's writes to shared memory visible to the tensor cores and TMA (the async proxy).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 64 consecutive columns of this warp's 32 tensor-memory lanes (lane i of the warp reads lane base + i).
__device__ __forceinline__ void tmem_load64(unsigned taddr, float (&v)[64]) {
    unsigned r[64];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]),
          "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]),
          "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]),
          "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 consecutive columns of this warp's 32 tensor-memory lanes, read and written back.
__device__ __forceinline__ void tmem_load32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\ttcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_store32(unsigned taddr, const float (&v)[32]) {
    unsigned r[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(v[i]);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
// 32 consecutive 32-bit columns of this warp's lanes, written as they are (packed pairs of 16-bit values for instance).
__device__ __forceinline__ void tmem_store32_words(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
// D (tensor memory) += A (tensor memory: rows on the lanes, pairs of 16-bit values along K in each 32-bit column) · B
// (shared memory, by descriptor).
__device__ __forceinline__ void tcgen05_mma_f16_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                                   unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of an MN-major tile ([k][n], n contiguous) in 128-byte swizzled rows of 64
// elements: 1024 bytes between groups of eight k, `chunk_bytes` between successive 64-element spans of n.
__device__ __forceinline__ unsigned long long umma_desc_sw128_mn(unsigned smem_addr, unsigned chunk_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((chunk_bytes >> 4) & 0x3FFFu) << 16;     // bits 16-29: leading-dimension byte offset / 16
    d |= (unsigned long long)(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// ------------------------------------------------------------------ host side: tensor maps
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

// A bfloat16 tensor of `rank` dimensions (innermost first; strides in bytes for dimensions 1...) read in boxes
// whose innermost extent is 64 elements, with the 128-byte swizzle; reads outside the tensor give zeros.
static int make_tensor_map(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                           const cuuint32_t* box) {
    PFN_cuTensorMapEncodeTiled fn = encode_tiled();
    if (fn == nullptr) return MLC_ERR_UNSUPPORTED;
    cuuint32_t elem[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : MLC_ERR_BAD_SIZE;
}

// The map of a row-major bfloat16 matrix [rows][cols] read in boxes of box_rows x box_cols, remembered by what defines
// it: a step launches hundreds of products over the same weights, and its scratch tensors come back at the same
// addresses step after step, so the driver is asked once per matrix, not once per launch.
static int cached_map_2d(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_cols, int box_rows) {
    struct Key {
        const void* ptr;
        long long rows, cols;
        int box_cols, box_rows;
        bool operator==(const Key& o) const {
            return ptr == o.ptr && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows;
        }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            size_t h = std::hash<const void*>()(k.ptr);
            h = h * 1000003u ^ std::hash<long long>()(k.rows * 131 + k.cols);
            return h * 1000003u ^ std::hash<int>()(k.box_cols * 1024 + k.box_rows);
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    static std::mutex lock;
    const Key key{ptr, rows, cols, box_cols, box_rows};
    {
        std::lock_guard<std::mutex> guard(lock);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return 0;
        }
    }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const int rc = make_tensor_map(map, ptr, 2, dims, strides, box);
    if (rc == 0) {
        std::lock_guard<std::mutex> guard(lock);
        if (cache.size() > 8192) cache.clear();
        cache.emplace(key, *map);
    }
    return rc;
}

}  // namespace mlc

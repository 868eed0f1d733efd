// What the tcgen05 products share: barriers with bounded waits, TMA copies, MMA issue, operand and
// instruction descriptors, and the tensor maps of [rows, K] bfloat16 matrices.
#pragma once
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace bg {

constexpr int TC_BM = 128;                 // output features per CTA (MMA M)
constexpr int TC_BK = 64;                  // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_THREADS = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr unsigned long long TC_WAIT_NS = 1000000000ull;   // a wait gives up after one second

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    unsigned addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        // the hint lets the hardware park the thread (up to 2 us) instead of polling: polls of many waiting
        // threads would crowd the shared-memory pipeline that the copies of other warps need
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(addr), "r"(parity), "r"(2000u) : "memory");
        if (done) return true;
        if ((it & 15u) == 15u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > TC_WAIT_NS) return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Thread block clusters: the cluster-wide barrier (every thread of every CTA arrives) and stores into a
// peer CTA's shared memory.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
// (nothing that this thread wrote has to be visible to the peers at the first use of the barrier)
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    cluster_arrive();
    cluster_wait();
}
// the address, in the cluster's shared window, of this CTA's shared-memory address in the CTA of the given rank
__device__ __forceinline__ unsigned peer_addr(unsigned local_addr, unsigned rank) {
    unsigned a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void st_cluster(unsigned addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes, 128-byte swizzle; groups
// of 8 rows are 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);          // start address
    d |= (unsigned long long)(1024u >> 4) << 32;                     // stride between 8-row groups
    d |= 1ull << 46;                                                 // descriptor version of sm_100
    d |= 2ull << 61;                                                 // 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: float accumulator, bfloat16 A and B, both K-major, M x N.
__host__ __device__ constexpr unsigned instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A [rows, K] bfloat16 matrix with row stride ld (elements), cut into boxes of box_rows x 64.
inline int make_map(CUtensorMap* map, const void* base, long long rows, int K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return BG_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BG_OK : BG_ERR_SHAPE;
}

// A [rows, cols] float matrix with row stride ld (elements), cut into boxes of box_rows x 32 (rows of 128 bytes).
inline int make_map_f32(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return BG_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? BG_OK : BG_ERR_SHAPE;
}

// The map of a weight matrix (boxes of box_rows x 64), made once per (pointer, shape, box) and kept.
inline int weight_map(CUtensorMap* out, const void* W, int n_out, int K, int ldw, int box_rows = TC_BM) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> w_maps;
    std::lock_guard<std::mutex> g(mu);
    auto key = std::make_tuple(W, n_out, K, ldw, box_rows);
    auto it = w_maps.find(key);
    if (it == w_maps.end()) {
        CUtensorMap mw;
        int rc = make_map(&mw, W, n_out, K, ldw, box_rows);
        if (rc != BG_OK) return rc;
        it = w_maps.emplace(key, mw).first;
    }
    *out = it->second;
    return BG_OK;
}

}  // namespace bg

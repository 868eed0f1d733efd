// Pages of the cache by TMA: the pool of one layer, [num_pages][2][nkv][page_size][head_dim] bfloat16,
// seen as a 2-D tensor of rows of head_dim features.  A box is one page of one kv head, 64 features
// wide, and lands in shared memory with the 128-byte swizzle: row j of the box at j * 128 bytes, its
// 16-byte piece c at ((c ^ (j & 7)) * 16).  Shared by the attention kernels that copy pages this way.
#pragma once
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace bg {

constexpr unsigned long long PT_WAIT_NS = 1000000000ull;     // a wait on a barrier gives up after a second

__device__ __forceinline__ unsigned pt_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pt_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(pt_smem(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void pt_mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void pt_mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(pt_smem(bar)) : "memory");
}
__device__ __forceinline__ void pt_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(pt_smem(bar)), "r"(bytes) : "memory");
}
// Adds to the bytes that the current phase waits for, without arriving.
__device__ __forceinline__ void pt_expect_only(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(pt_smem(bar)), "r"(bytes) : "memory");
}
// Waits for the phase of the given parity; gives up after PT_WAIT_NS, or as soon as *gave_up (a flag in
// shared memory that the first thread to give up sets) is non-zero, and returns false then.
__device__ __forceinline__ bool pt_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* gave_up) {
    const unsigned addr = pt_smem(bar);
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
        unsigned done;
        // the time hint parks the thread in hardware for up to that long instead of polling: the polls of a
        // hundred waiting threads crowd the pipeline that the copies of the issuing warp go through
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(addr), "r"(parity), "r"(4000u) : "memory");
        if (done) return true;
        if ((it & 15u) == 15u) {
            if (gave_up && *gave_up) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > PT_WAIT_NS) { if (gave_up) *gave_up = 1; return false; }
        }
    }
}
__device__ __forceinline__ void pt_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(pt_smem(dst)), "l"(map), "r"(x), "r"(y), "r"(pt_smem(bar)) : "memory");
}
// The keys AND values of one page of one kv head in one copy (see pt_page_map): u = page * 2 * nkv + kv head.
__device__ __forceinline__ void pt_tma_page(void* dst, const CUtensorMap* map, int u, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %2, %2, %2, %3}], [%4];\n"
                 ::"r"(pt_smem(dst)), "l"(map), "r"(0), "r"(u), "r"(pt_smem(bar)) : "memory");
}
__device__ __forceinline__ void pt_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(map) : "memory");
}
__device__ __forceinline__ void pt_fence_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Whether pages of this size can be copied as boxes into tiles of 64 keys.
inline bool pt_page_size_ok(int page_size) { return page_size >= 1 && page_size <= 64 && 64 % page_size == 0; }

// The tensor map of a pool, made once per (pointer, shape) and kept.
inline int pt_pool_map(CUtensorMap* out, const void* pool, int num_pages, int nkv, int page_size, int hd) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> maps;
    static EncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeFn)f;
    }();
    if (!fn || !pt_page_size_ok(page_size) || hd % 64 != 0) return BG_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> g(mu);
    const auto key = std::make_tuple(pool, num_pages, nkv, page_size, hd);
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap map;
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)num_pages * 2 * nkv * page_size};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return BG_ERR_SHAPE;
        it = maps.emplace(key, map).first;
    }
    *out = it->second;
    return BG_OK;
}

// A second view of the same pool, for whole pages: five dimensions (64 features | the page's rows | the
// blocks of 64 features of a row | keys, values | page and kv head), so that ONE box is everything a kv
// head has in a page.  It lands as [keys, values][block of 64 features][row][128 bytes, swizzled]: for a
// page of 64 positions exactly a tile of 64 keys and one of 64 values in the layout above.  (What costs
// the issuing thread is the copy instruction, not the bytes it moves.)
inline int pt_page_map(CUtensorMap* out, const void* pool, int num_pages, int nkv, int page_size, int hd) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> maps;
    static EncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (EncodeFn)f;
    }();
    if (!fn || !pt_page_size_ok(page_size) || hd % 64 != 0 || page_size * (hd / 64) * 2 * 128 > 65536) return BG_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> g(mu);
    const auto key = std::make_tuple(pool, num_pages, nkv, page_size, hd);
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap map;
        const cuuint64_t slab = (cuuint64_t)page_size * hd * 2;      // bytes of one (page, keys or values, kv head)
        cuuint64_t dims[5] = {64, (cuuint64_t)page_size, (cuuint64_t)hd / 64, 2, (cuuint64_t)num_pages * 2 * nkv - nkv};
        cuuint64_t strides[4] = {(cuuint64_t)hd * 2, 128, (cuuint64_t)nkv * slab, slab};
        cuuint32_t box[5] = {64, (cuuint32_t)page_size, (cuuint32_t)hd / 64, 2, 1};
        cuuint32_t elem[5] = {1, 1, 1, 1, 1};
        CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(pool), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return BG_ERR_SHAPE;
        it = maps.emplace(key, map).first;
    }
    *out = it->second;
    return BG_OK;
}

}  // namespace bg

// Pages of the cache by TMA: the pool of one layer, [num_pages][2][nkv][page_size][head_dim] bfloat16,
// seen as a 2-D tensor of rows of head_dim features.  A box is one page of one kv head, 64 features
// wide, and lands in shared memory with the 128-byte swizzle: row j of the box at j * 128 bytes, its
// 16-byte piece c at ((c ^ (j & 7)) * 16).  Shared by the attention kernels that copy pages this way.
#pragma once
#include <map>
#include <mutex>
#include <tuple>

#include "ptx.cuh"

namespace bg {

// Whether pages of this size can be copied as boxes into tiles of 64 keys.
inline bool pt_page_size_ok(int page_size) { return page_size >= 1 && page_size <= 64 && 64 % page_size == 0; }

// The tensor map of a pool, made once per (pointer, shape) and kept.
inline int pt_pool_map(CUtensorMap* out, const void* pool, int num_pages, int nkv, int page_size, int hd) {
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> maps;
    const EncodeTiledFn fn = encode_fn();
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
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> maps;
    const EncodeTiledFn fn = encode_fn();
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

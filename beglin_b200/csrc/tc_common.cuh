// What the tcgen05 products share beyond the PTX wrappers of ptx.cuh: tile constants, the helpers of thread block
// clusters, and the tensor maps of [rows, K] matrices.
#pragma once
#include <map>
#include <mutex>
#include <tuple>

#include "ptx.cuh"

namespace bg {

constexpr int TC_BM = 128;                 // output features per CTA (MMA M)
constexpr int TC_BK = 64;                  // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_THREADS = 192;            // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue

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

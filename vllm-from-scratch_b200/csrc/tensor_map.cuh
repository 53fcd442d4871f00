// Tensor maps (TMA descriptors) for row-major bfloat16 matrices, made with the driver's
// encoder, which is found through the runtime so that nothing links against libcuda.
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace b200 {

constexpr int kTensorMapBoxColumns = 64;      // 128 bytes of bfloat16: one swizzle row

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, found through the runtime (no link against libcuda).
inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* found = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &found, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(found);
    }
    return fn;
}

// Tensor map of a row-major bfloat16 matrix [rows, K] with boxes of 64 columns (128 bytes,
// swizzled) x box_rows rows; rows outside the matrix read as zeros.  Maps are cached by
// (address, rows, K, box_rows): weights keep theirs for the life of the process.
inline const CUtensorMap* tensor_map_for(const void* base, int rows, int K, int box_rows) {
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    const auto key = std::make_tuple(base, rows, K, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) return &it->second;
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) return nullptr;
    if (cache.size() > 4096) cache.clear();
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTensorMapBoxColumns, (cuuint32_t)box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                   box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) return nullptr;
    return &cache.emplace(key, map).first->second;
}

}  // namespace b200

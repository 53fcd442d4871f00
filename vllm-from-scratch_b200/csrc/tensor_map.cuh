// Tensor maps (TMA descriptors) for row-major bfloat16 matrices, made with the driver's
// encoder, which is found through the runtime so that nothing links against libcuda.
#pragma once

#include <cuda.h>

#include <cstring>
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
//
// The map is copied into *out while the lock is held, so a caller never holds a pointer
// into the cache: a launcher looks up two or three maps in a row, and a later look-up (its
// own, or another thread's) may empty a full cache.  Returns false if the driver's encoder
// is missing or refuses the shape.
constexpr size_t kTensorMapCacheLimit = 4096;

inline bool tensor_map_for(const void* base, int rows, int K, int box_rows, CUtensorMap* out) {
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    const auto key = std::make_tuple(base, rows, K, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) return false;
    // Maps of activations are keyed by an address that changes from step to step, so the
    // cache fills in a long run without graphs; nobody holds a pointer into it, so it may go.
    if (cache.size() >= kTensorMapCacheLimit) cache.clear();
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTensorMapBoxColumns, (cuuint32_t)box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult status = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                                   box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) return false;
    cache.emplace(key, map);
    *out = map;
    return true;
}

// Host-only check of the cache's lifetime rule (no kernel is launched, the addresses are only
// encoded): takes maps of `count` different addresses inside [base, base + bytes), more than
// the cache holds, keeps the first copies, and compares them byte for byte with maps taken
// again after the cache has been emptied under them.  Returns 0 if all agree, a positive
// count of mismatches, or -1 if a map could not be encoded.
inline int tensor_map_cache_self_check(const void* base, size_t bytes, int count) {
    const int rows = 64, K = 64, box_rows = 8, kept = 8;
    const size_t step = 16;
    if ((size_t)count * step + (size_t)rows * K * 2 > bytes) return -1;
    CUtensorMap first[kept];
    const char* start = static_cast<const char*>(base);
    for (int i = 0; i < count; ++i) {
        CUtensorMap map;
        if (!tensor_map_for(start + (size_t)i * step, rows, K, box_rows, &map)) return -1;
        if (i < kept) first[i] = map;
    }
    int mismatches = 0;
    for (int i = 0; i < kept && i < count; ++i) {
        CUtensorMap again;
        if (!tensor_map_for(start + (size_t)i * step, rows, K, box_rows, &again)) return -1;
        if (memcmp(&again, &first[i], sizeof(CUtensorMap)) != 0) ++mismatches;
    }
    return mismatches;
}

}  // namespace b200

// Shared helpers of the sm_100a kernels: element conversion, warp and block
// reductions, launch-error reporting.  Every launcher is `extern "C"`, takes raw
// device pointers and a stream, and returns 0 or a negative code after storing a
// message that `b200_last_error` hands to the Python side.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define B200_EXPORT extern "C" __attribute__((visibility("default")))

namespace b200 {

inline char* error_buffer() {
    static thread_local char buffer[512];
    return buffer;
}

inline int fail(const char* where, const char* what) {
    snprintf(error_buffer(), 512, "%s: %s", where, what);
    return -1;
}

inline int check_launch(const char* where) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(where, cudaGetErrorString(status));
    return 0;
}

// Number of SMs of the calling thread's device, asked of the device once; 0 if it cannot be read.
// Launch planning (how many blocks fill the GPU) uses this, never a literal.
inline int sm_count() {
    static int count[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
    if (count[device] == 0) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
        count[device] = value;
    }
    return count[device];
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Rotation of a pair of channels by an angle (rotate-half position encoding).  Written out
// with the product that is rounded on its own named, because a compiler may contract
// a * b - c * d either way: every kernel that rotates (for a portion of a prompt, for a decode
// step, inside the decode attention) must round a key or a query alike.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float c, float s, float& o1, float& o2) {
    o1 = fmaf(x1, c, -__fmul_rn(x2, s));
    o2 = fmaf(x2, c, __fmul_rn(x1, s));
}

// Sum over the whole block; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float total = lane < warps ? scratch[lane] : 0.0f;
        total = warp_sum(total);
        if (lane == 0) scratch[32] = total;
    }
    __syncthreads();
    float result = scratch[32];
    __syncthreads();
    return result;
}

// ---------------------------------------------------------------- overlapped launches
// A decode step is a chain of some hundred short kernels.  Launched "overlapped"
// (programmatic dependent launch), a kernel may be scheduled while its predecessor on
// the stream is still draining: it runs up to `overlap_wait()` (which returns when the
// predecessor has completed and its writes are visible), so everything before that
// call (index arithmetic, barrier and tensor-memory set-up, loads of weights, which
// no kernel writes) overlaps the predecessor's tail.  `overlap_trigger()` tells the
// scheduler that the kernels after this one may start being scheduled.
// A kernel launched this way must not read anything a predecessor writes, nor write
// anything at all, before `overlap_wait()`.
__device__ __forceinline__ void overlap_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void overlap_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

inline bool overlap_enabled() {
    static const bool enabled = getenv("B200_NO_OVERLAP") == nullptr;
    return enabled;
}

template <typename... Params, typename... Args>
inline void launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = overlap_enabled() ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

}  // namespace b200

// One translation unit per shared object, so this definition appears once in each.
B200_EXPORT const char* b200_last_error() { return b200::error_buffer(); }

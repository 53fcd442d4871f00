// Embedding gather and RMSNorm with the residual sum fused in.
//
// The residual stream is float32 in both run modes.  One block per row:
//   pass 1: v = residual + x (x optional), stored back unless rows are gathered,
//           sum of squares accumulated in float32;
//   pass 2: out = v * rsqrt(mean(v^2) + eps) * weight, rounded once to the run dtype.
// Formula: minivllm/layers/ops/layernorm.py:196-227 (epsilon inside the root, no
// bias, plain weight); the sum and the statistics stay in 32-bit as in
// minivllm/layers/ops/layernorm.py:75-90.
#include "common.cuh"

namespace b200 {

template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, float* __restrict__ residual,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    const int out_row = blockIdx.x;
    const int row = rows ? rows[out_row] : out_row;
    const size_t base = (size_t)row * hidden;
    const bool store_sum = (rows == nullptr) && (x != nullptr);
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = residual[base + i];
        if (x) v += to_float(x[base + i]);
        if (store_sum) residual[base + i] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    const float total = block_sum(sum_sq, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    const size_t out_base = (size_t)out_row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = residual[base + i];
        if (x && !store_sum) v += to_float(x[base + i]);
        out[out_base + i] = from_float<T>(v * inv * weight[i]);
    }
}

// Four elements per thread and step with 8- or 16-byte accesses; the row's sums stay in
// registers between the two passes (up to four steps: rows up to 16 * blockDim wide).
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&a);
        raw.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// EARLY (launches of a few rows, where the kernel is one round trip long): the norm's weights,
// which no kernel writes, are fetched before the wait for the kernel ahead instead of after the
// reduction.  Launches of many rows keep the registers for more blocks per SM.
template <typename T, bool EARLY>
__global__ void add_rmsnorm_vec_kernel(const T* __restrict__ x, float* __restrict__ residual,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    constexpr int kSteps = 4;
    overlap_trigger();
    const int out_row = blockIdx.x;
    float4 scale[EARLY ? kSteps : 1];
    if (EARLY) {
#pragma unroll
        for (int step = 0; step < kSteps; ++step) {
            const int i = (step * blockDim.x + threadIdx.x) * 4;
            scale[step] = i < hidden ? *reinterpret_cast<const float4*>(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    overlap_wait();
    const int row = rows ? rows[out_row] : out_row;
    const size_t base = (size_t)row * hidden;
    const bool store_sum = (rows == nullptr) && (x != nullptr);
    float4 kept[kSteps];
    float sum_sq = 0.0f;
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            float4 v = *reinterpret_cast<const float4*>(residual + base + i);
            if (x) {
                const float4 add = Vec4<T>::load(x + base + i);
                v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
            }
            if (store_sum) *reinterpret_cast<float4*>(residual + base + i) = v;
            sum_sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            kept[step] = v;
        }
    }
    const float total = block_sum(sum_sq, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    const size_t out_base = (size_t)out_row * hidden;
#pragma unroll
    for (int step = 0; step < kSteps; ++step) {
        const int i = (step * blockDim.x + threadIdx.x) * 4;
        if (i < hidden) {
            const float4 w = EARLY ? scale[EARLY ? step : 0] : *reinterpret_cast<const float4*>(weight + i);
            const float4 v = kept[step];
            Vec4<T>::store(out + out_base + i, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
        }
    }
}

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ residual, int hidden, int vocab,
                                 int* __restrict__ error_flag) {
    const int token = blockIdx.x;
    const int id = ids[token];
    if (id < 0 || id >= vocab) {
        // A token id outside the table: record it and write zeros instead of reading.
        if (threadIdx.x == 0) atomicExch(error_flag, token + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) residual[(size_t)token * hidden + i] = 0.0f;
        return;
    }
    const T* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        residual[(size_t)token * hidden + i] = to_float(src[i]);
}

// Eight elements per thread with 16-byte accesses (bfloat16) or four with 16 bytes (float32).
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
    constexpr int kPer = 16 / sizeof(T);
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * kPer;
    if (i >= inter) return;
    const size_t token = blockIdx.y;
    const T* g = gate_up + token * 2 * inter + i;
    const uint4 graw = *reinterpret_cast<const uint4*>(g);
    const uint4 uraw = *reinterpret_cast<const uint4*>(g + inter);
    const T* gv = reinterpret_cast<const T*>(&graw);
    const T* uv = reinterpret_cast<const T*>(&uraw);
    uint4 result;
    T* rv = reinterpret_cast<T*>(&result);
#pragma unroll
    for (int e = 0; e < kPer; ++e) {
        const float gf = to_float(gv[e]);
        rv[e] = from_float<T>(gf / (1.0f + expf(-gf)) * to_float(uv[e]));
    }
    *reinterpret_cast<uint4*>(out + token * inter + i) = result;
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
    // out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i], all in float32.
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t token = idx / inter;
        const int i = (int)(idx - token * inter);
        const float g = to_float(gate_up[token * 2 * inter + i]);
        const float u = to_float(gate_up[token * 2 * inter + inter + i]);
        const float s = g / (1.0f + expf(-g));
        out[idx] = from_float<T>(s * u);
    }
}

inline int norm_threads(int hidden) {
    int threads = 128;
    while (threads < 1024 && threads * 4 < hidden) threads *= 2;
    return threads;
}

}  // namespace b200

// dtype: 0 = float32, 1 = bfloat16 (the dtype of x and out; residual and weight are float32).
B200_EXPORT int b200_add_rmsnorm(const void* x, float* residual, const float* weight, void* out,
                                 const int* rows, int num_rows, int hidden, float eps, int dtype,
                                 cudaStream_t stream) {
    using namespace b200;
    if (num_rows == 0) return 0;
    if (num_rows < 0 || hidden <= 0) return fail("add_rmsnorm", "negative row count or width");
    if (dtype != 0 && dtype != 1) return fail("add_rmsnorm", "dtype must be 0 (float32) or 1 (bfloat16)");
    const uintptr_t addresses = (uintptr_t)x | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out;
    if (hidden % 4 == 0 && hidden <= 16 * 1024 && (addresses & 15) == 0) {
        int threads = 64;
        while (threads < 1024 && threads * 16 < hidden) threads *= 2;      // at most four steps a thread
        while (threads < 256 && threads * 4 < hidden) threads *= 2;        // short rows: one step a thread
        const bool early = num_rows <= 64;
        if (dtype == 0 && early)
            launch_overlapped(add_rmsnorm_vec_kernel<float, true>, num_rows, threads, 0, stream,
                              (const float*)x, residual, weight, (float*)out, rows, hidden, eps);
        else if (dtype == 0)
            launch_overlapped(add_rmsnorm_vec_kernel<float, false>, num_rows, threads, 0, stream,
                              (const float*)x, residual, weight, (float*)out, rows, hidden, eps);
        else if (early)
            launch_overlapped(add_rmsnorm_vec_kernel<__nv_bfloat16, true>, num_rows, threads, 0, stream,
                              (const __nv_bfloat16*)x, residual, weight, (__nv_bfloat16*)out, rows, hidden, eps);
        else
            launch_overlapped(add_rmsnorm_vec_kernel<__nv_bfloat16, false>, num_rows, threads, 0, stream,
                              (const __nv_bfloat16*)x, residual, weight, (__nv_bfloat16*)out, rows, hidden, eps);
        return check_launch("add_rmsnorm");
    }
    const int threads = norm_threads(hidden);
    if (dtype == 0)
        add_rmsnorm_kernel<float><<<num_rows, threads, 0, stream>>>(
            (const float*)x, residual, weight, (float*)out, rows, hidden, eps);
    else
        add_rmsnorm_kernel<__nv_bfloat16><<<num_rows, threads, 0, stream>>>(
            (const __nv_bfloat16*)x, residual, weight, (__nv_bfloat16*)out, rows, hidden, eps);
    return check_launch("add_rmsnorm");
}

B200_EXPORT int b200_embedding(const void* table, const int* ids, float* residual, int num_tokens,
                               int hidden, int vocab, int* error_flag, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    const int threads = norm_threads(hidden);
    if (dtype == 0)
        embedding_kernel<float><<<num_tokens, threads, 0, stream>>>(
            (const float*)table, ids, residual, hidden, vocab, error_flag);
    else if (dtype == 1)
        embedding_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(
            (const __nv_bfloat16*)table, ids, residual, hidden, vocab, error_flag);
    else
        return fail("embedding", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("embedding");
}

B200_EXPORT int b200_silu_mul(const void* gate_up, void* out, int num_tokens, int inter, int dtype,
                              cudaStream_t stream) {
    using namespace b200;
    const size_t total = (size_t)num_tokens * inter;
    if (total == 0) return 0;
    if (dtype != 0 && dtype != 1) return fail("silu_mul", "dtype must be 0 (float32) or 1 (bfloat16)");
    const int per = dtype == 0 ? 4 : 8;
    if (inter % per == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0 && num_tokens <= 65535) {
        dim3 grid((inter / per + 255) / 256, num_tokens);
        if (dtype == 0)
            silu_mul_vec_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter);
        else
            silu_mul_vec_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
                (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
        return check_launch("silu_mul");
    }
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)(sm_count() > 0 ? sm_count() : 1) * 32;
    if (blocks > most) blocks = most;
    if (dtype == 0)
        silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
    else if (dtype == 1)
        silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else
        return fail("silu_mul", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("silu_mul");
}

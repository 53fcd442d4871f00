// Per-head RMSNorm of queries and keys, rotate-half position encoding, and the
// write of keys and values into their pages: one pass over the packed projection.
//
// Input  qkv  [T, (nq + 2 nkv) d]  rows = [queries | keys | values]
// Output q    [T, nq d]            normalised and rotated queries
//        K, V pages [pages, nkv, page_size, d] at slot = page * page_size + offset
//
// Order of operations as in minivllm/models/qwen3.py:111-117 (norm over the head
// dimension with one weight vector shared by all heads, then rotation, values
// untouched) and minivllm/layers/ops/rotary_embedding.py:243-257 (x1 = first
// half, x2 = second half; o1 = x1 cos - x2 sin, o2 = x2 cos + x1 sin).  The angle
// is position * inv_freq in float32 with the precise sincosf; statistics in
// float32.  A negative slot means "do not store" (minivllm/attention/ops/
// triton_reshape_and_cache_flash.py:43-85).
#include "common.cuh"

namespace b200 {

template <typename T>
__global__ void head_norm_rope_cache_kernel(
    const T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    const float* __restrict__ inv_freq, T* __restrict__ q_out, T* __restrict__ k_pages,
    T* __restrict__ v_pages, int nq, int nkv, int d, int rotary_dim, int page_size, float eps) {
    overlap_trigger();
    overlap_wait();
    const int token = blockIdx.x;
    const int warps = blockDim.x >> 5;
    const int head_slot = blockIdx.y * warps + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int total_heads = nq + 2 * nkv;
    if (head_slot >= total_heads) return;
    const bool is_q = head_slot < nq;
    const bool is_k = !is_q && head_slot < nq + nkv;
    const bool is_v = !is_q && !is_k;
    if (!is_q && k_pages == nullptr) return;  // this execution owns no cache: keys/values unused

    const T* src = qkv + (size_t)token * total_heads * d + (size_t)head_slot * d;
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)token * nq * d + (size_t)head_slot * d;
    } else {
        const int slot = slots[token];
        if (slot < 0) return;
        const int page = slot / page_size, offset = slot - page * page_size;
        const int kv_head = is_k ? head_slot - nq : head_slot - nq - nkv;
        T* pages = is_k ? k_pages : v_pages;
        dst = pages + (((size_t)page * nkv + kv_head) * page_size + offset) * d;
    }
    if (is_v) {
        for (int j = lane; j < d; j += 32) dst[j] = src[j];
        return;
    }
    const float* weight = is_q ? q_weight : k_weight;
    float inv = 1.0f;
    if (weight) {
        float sum_sq = 0.0f;
        for (int j = lane; j < d; j += 32) {
            const float v = to_float(src[j]);
            sum_sq = fmaf(v, v, sum_sq);
        }
        sum_sq = warp_sum(sum_sq);
        inv = rsqrtf(sum_sq / (float)d + eps);
    }
    const int half = rotary_dim >> 1;
    const float pos = (float)positions[token];
    for (int j = lane; j < half; j += 32) {
        float x1 = to_float(src[j]) * inv, x2 = to_float(src[j + half]) * inv;
        if (weight) { x1 *= weight[j]; x2 *= weight[j + half]; }
        float s, c;
        sincosf(pos * inv_freq[j], &s, &c);
        dst[j] = from_float<T>(x1 * c - x2 * s);
        dst[j + half] = from_float<T>(x2 * c + x1 * s);
    }
    for (int j = rotary_dim + lane; j < d; j += 32) {
        float v = to_float(src[j]) * inv;
        if (weight) v *= weight[j];
        dst[j] = from_float<T>(v);
    }
}

}  // namespace b200

// dtype: 0 = float32, 1 = bfloat16.  q_weight / k_weight may be null (no head
// norm), inv_freq may be null with rotary_dim = 0 (no rotation), k_pages / v_pages
// may be null (nothing is stored).
B200_EXPORT int b200_head_norm_rope_cache(
    const void* qkv, const int* positions, const int* slots, const float* q_weight,
    const float* k_weight, const float* inv_freq, void* q_out, void* k_pages, void* v_pages,
    int num_tokens, int nq, int nkv, int d, int rotary_dim, int page_size, float eps, int dtype,
    cudaStream_t stream) {
    using namespace b200;
    if (num_tokens == 0) return 0;
    if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1))
        return fail("head_norm_rope_cache", "rotary_dim must be even and at most head_dim");
    if (rotary_dim > 0 && inv_freq == nullptr)
        return fail("head_norm_rope_cache", "rotation asked for without inverse frequencies");
    if ((k_pages == nullptr) != (v_pages == nullptr))
        return fail("head_norm_rope_cache", "key and value pages must be given together");
    if (k_pages && page_size <= 0) return fail("head_norm_rope_cache", "page_size must be positive");
    const int warps = 4;
    const int total_heads = nq + 2 * nkv;
    dim3 grid(num_tokens, (total_heads + warps - 1) / warps);
    if (grid.y > 65535) return fail("head_norm_rope_cache", "too many heads");
    if (dtype == 0)
        launch_overlapped(head_norm_rope_cache_kernel<float>, grid, warps * 32, 0, stream,
            (const float*)qkv, positions, slots, q_weight, k_weight, inv_freq, (float*)q_out,
            (float*)k_pages, (float*)v_pages, nq, nkv, d, rotary_dim, page_size, eps);
    else if (dtype == 1)
        launch_overlapped(head_norm_rope_cache_kernel<__nv_bfloat16>, grid, warps * 32, 0, stream,
            (const __nv_bfloat16*)qkv, positions, slots, q_weight, k_weight, inv_freq,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, nq, nkv, d,
            rotary_dim, page_size, eps);
    else
        return fail("head_norm_rope_cache", "dtype must be 0 (float32) or 1 (bfloat16)");
    return check_launch("head_norm_rope_cache");
}

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

    // Everything that does not come from the kernel before this one is fetched and worked out
    // before waiting for it: position and slot (inputs of the step), the angles' sines and
    // cosines, the norm weights.  After the wait only the head itself is read.
    constexpr int kMaxPairs = 8;                    // pairs of channels per lane held in registers
    const int half = rotary_dim >> 1;
    const bool held = half <= 32 * kMaxPairs;
    const float* weight = is_q ? q_weight : k_weight;
    const float pos = (float)positions[token];
    int slot = 0;
    if (!is_q) {
        slot = slots[token];
        if (slot < 0) return;
    }
    float sin_r[kMaxPairs], cos_r[kMaxPairs], w1_r[kMaxPairs], w2_r[kMaxPairs];
    if (!is_v && held) {
#pragma unroll
        for (int i = 0; i < kMaxPairs; ++i) {
            const int j = lane + 32 * i;
            sin_r[i] = 0.0f; cos_r[i] = 1.0f; w1_r[i] = w2_r[i] = 1.0f;
            if (j < half) {
                sincosf(pos * inv_freq[j], &sin_r[i], &cos_r[i]);
                if (weight) { w1_r[i] = weight[j]; w2_r[i] = weight[j + half]; }
            }
        }
    }
    const T* src = qkv + (size_t)token * total_heads * d + (size_t)head_slot * d;
    T* dst;
    if (is_q) {
        dst = q_out + (size_t)token * nq * d + (size_t)head_slot * d;
    } else {
        const int page = slot / page_size, offset = slot - page * page_size;
        const int kv_head = is_k ? head_slot - nq : head_slot - nq - nkv;
        T* pages = is_k ? k_pages : v_pages;
        dst = pages + (((size_t)page * nkv + kv_head) * page_size + offset) * d;
    }
    overlap_wait();

    if (is_v) {
        for (int j = lane; j < d; j += 32) dst[j] = src[j];
        return;
    }
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
    if (held) {
#pragma unroll
        for (int i = 0; i < kMaxPairs; ++i) {
            const int j = lane + 32 * i;
            if (j < half) {
                const float x1 = to_float(src[j]) * inv * w1_r[i], x2 = to_float(src[j + half]) * inv * w2_r[i];
                float o1, o2;
                rotate_pair(x1, x2, cos_r[i], sin_r[i], o1, o2);
                dst[j] = from_float<T>(o1);
                dst[j + half] = from_float<T>(o2);
            }
        }
    } else {
        for (int j = lane; j < half; j += 32) {
            float x1 = to_float(src[j]) * inv, x2 = to_float(src[j + half]) * inv;
            if (weight) { x1 *= weight[j]; x2 *= weight[j + half]; }
            float s, c;
            sincosf(pos * inv_freq[j], &s, &c);
            float o1, o2;
            rotate_pair(x1, x2, c, s, o1, o2);
            dst[j] = from_float<T>(o1);
            dst[j + half] = from_float<T>(o2);
        }
    }
    for (int j = rotary_dim + lane; j < d; j += 32) {
        float v = to_float(src[j]) * inv;
        if (weight) v *= weight[j];
        dst[j] = from_float<T>(v);
    }
}

// The same work for many tokens at once (portions of prompts), bfloat16, rotation over the
// whole head: one block per token.  The token's sines and cosines are computed once and
// shared by all of its heads through shared memory; half a warp owns a head, each lane
// PER elements of the first half and the matching PER of the second, read and written as
// one vector each.
template <int D>
__global__ void __launch_bounds__(128) head_norm_rope_cache_token_kernel(
    const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slots,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages,
    __nv_bfloat16* __restrict__ v_pages, int nq, int nkv, int page_size, float eps) {
    constexpr int HALF = D / 2, PER = HALF / 16;
    struct alignas(2 * PER) Vec { __nv_bfloat16 v[PER]; };
    __shared__ float sin_s[HALF], cos_s[HALF];
    overlap_trigger();              // the attention kernel behind this one may set itself up meanwhile
    const int token = blockIdx.x;
    const float pos = (float)positions[token];
    for (int j = threadIdx.x; j < HALF; j += blockDim.x) sincosf(pos * inv_freq[j], &sin_s[j], &cos_s[j]);
    __syncthreads();
    const int half_warp = threadIdx.x >> 4, sub = threadIdx.x & 15;
    const int total_heads = nq + 2 * nkv;
    const int slot = k_pages ? slots[token] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, offset = slot >= 0 ? slot - page * page_size : 0;
    const unsigned mask = 0xFFFFu << (threadIdx.x & 16);
    for (int head = half_warp; head < total_heads; head += 8) {
        const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
        if (!is_q && slot < 0) continue;                        // nothing is stored for this token
        const __nv_bfloat16* src = qkv + ((size_t)token * total_heads + head) * D + sub * PER;
        __nv_bfloat16* dst;
        if (is_q) {
            dst = q_out + ((size_t)token * nq + head) * D;
        } else {
            const int kv_head = is_k ? head - nq : head - nq - nkv;
            dst = (is_k ? k_pages : v_pages) + (((size_t)page * nkv + kv_head) * page_size + offset) * D;
        }
        dst += sub * PER;
        const Vec lo = *reinterpret_cast<const Vec*>(src), hi = *reinterpret_cast<const Vec*>(src + HALF);
        if (!is_q && !is_k) {                                   // values: copied as they are
            *reinterpret_cast<Vec*>(dst) = lo;
            *reinterpret_cast<Vec*>(dst + HALF) = hi;
            continue;
        }
        float x1[PER], x2[PER];
#pragma unroll
        for (int e = 0; e < PER; ++e) { x1[e] = __bfloat162float(lo.v[e]); x2[e] = __bfloat162float(hi.v[e]); }
        const float* weight = is_q ? q_weight : k_weight;
        if (weight) {
            float sum_sq = 0.0f;
#pragma unroll
            for (int e = 0; e < PER; ++e) sum_sq = fmaf(x1[e], x1[e], fmaf(x2[e], x2[e], sum_sq));
#pragma unroll
            for (int step = 8; step > 0; step >>= 1) sum_sq += __shfl_xor_sync(mask, sum_sq, step);
            const float inv = rsqrtf(sum_sq / (float)D + eps);
#pragma unroll
            for (int e = 0; e < PER; ++e) {
                x1[e] = x1[e] * inv * weight[sub * PER + e];
                x2[e] = x2[e] * inv * weight[HALF + sub * PER + e];
            }
        }
        Vec out_lo, out_hi;
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const float s = sin_s[sub * PER + e], c = cos_s[sub * PER + e];
            float o1, o2;
            rotate_pair(x1[e], x2[e], c, s, o1, o2);
            out_lo.v[e] = __float2bfloat16_rn(o1);
            out_hi.v[e] = __float2bfloat16_rn(o2);
        }
        *reinterpret_cast<Vec*>(dst) = out_lo;
        *reinterpret_cast<Vec*>(dst + HALF) = out_hi;
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
    // Many tokens: the kernel that shares a token's sines and cosines between its heads.
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    if (dtype == 1 && num_tokens >= 32 && rotary_dim == d && (d == 64 || d == 128 || d == 256) && aligned) {
#define B200_CASE(D)                                                                                     \
        if (d == D)                                                                                      \
            head_norm_rope_cache_token_kernel<D><<<num_tokens, 128, 0, stream>>>(                        \
                (const __nv_bfloat16*)qkv, positions, slots, q_weight, k_weight, inv_freq,              \
                (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, nq, nkv, page_size, eps);
        B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
        return check_launch("head_norm_rope_cache");
    }
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

// Paged causal attention with grouped query heads for any mix of query lengths:
// the float32-arithmetic kernel.  It is the whole attention of the true 32-bit
// run mode and the fallback of the bfloat16 mode for shapes the tensor-core
// kernels refuse.
//
// One block = 16 consecutive query tokens of one request x one query head.  The
// request of a block is found from its index alone (no host-side tile list):
// request r owns the block indices [query_start[r] / 16 + r, query_start[r+1] / 16
// + r + 1), an over-allocation of at most one block per request, the scheme of
// minivllm/attention/ops/triton_unified_attention.py:150-239.  Keys are read
// through the request's block table in tiles of 32 positions; scores, the running
// maximum and sum, and the output accumulate in float32 (online softmax); a row
// with no visible key yields zeros (minivllm/attention/ops/
// triton_unified_attention.py:390).
//
// Masking, with past = seq_len - q_len and query i at position past + i:
//   key position kp is visible iff kp <= past + i  (causal)
//                              and kp >  past + i - window  (when window > 0).
// minivllm/attention/backends/torch_sdpa.py:450-489 states the causal rule.
#include "common.cuh"

namespace b200 {

constexpr int kQueryTile = 16;
constexpr int kKeyTile = 32;
constexpr int kWarps = 4;
constexpr int kRowsPerWarp = kQueryTile / kWarps;

template <typename T, int DPL>  // DPL: head-dim elements per lane, head_dim <= 32 * DPL
__global__ void __launch_bounds__(kWarps * 32) paged_attention_generic_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
    T* __restrict__ out, const int* __restrict__ query_start, const int* __restrict__ seq_lens,
    const int* __restrict__ block_table, int num_requests, int max_pages, int nq, int nkv, int d,
    int page_size, float scale, int window) {
    extern __shared__ float smem[];
    float* q_s = smem;                                   // [16][d]
    float* k_s = q_s + kQueryTile * d;                   // [32][d + 1]
    float* v_s = k_s + kKeyTile * (d + 1);               // [32][d]

    // Which request does this block belong to?  Largest r with start[r]/16 + r <= block.
    const int block = blockIdx.x;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (query_start[mid] / kQueryTile + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int local_tile = block - (q_begin / kQueryTile + request);
    const int tile_first = local_tile * kQueryTile;
    if (tile_first >= q_len) return;
    const int rows_here = min(kQueryTile, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const int* table = block_table + (size_t)request * max_pages;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int idx = tid; idx < kQueryTile * d; idx += blockDim.x) {
        const int row = idx / d, j = idx - row * d;
        float v = 0.0f;
        if (row < rows_here)
            v = to_float(q[((size_t)(q_begin + tile_first + row) * nq + head) * d + j]);
        q_s[idx] = v;
    }

    float acc[kRowsPerWarp][DPL];
    float row_max[kRowsPerWarp], row_sum[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        row_max[r] = -INFINITY;
        row_sum[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }

    const int first_pos = past + tile_first;                 // position of the tile's first query
    const int last_pos = first_pos + rows_here - 1;
    int key_begin = 0;
    if (window > 0) key_begin = max(0, first_pos - window + 1);
    key_begin = (key_begin / kKeyTile) * kKeyTile;
    const int key_end = last_pos + 1;                        // causal: nothing beyond the last query

    for (int k0 = key_begin; k0 < key_end; k0 += kKeyTile) {
        __syncthreads();
        for (int idx = tid; idx < kKeyTile * d; idx += blockDim.x) {
            const int key = idx / d, j = idx - key * d;
            const int kp = k0 + key;
            float kv = 0.0f, vv = 0.0f;
            if (kp < key_end) {
                const int page = table[kp / page_size];
                if (page >= 0) {
                    const size_t at = (((size_t)page * nkv + kv_head) * page_size + kp % page_size) * d + j;
                    kv = to_float(k_pages[at]);
                    vv = to_float(v_pages[at]);
                }
            }
            k_s[key * (d + 1) + j] = kv;
            v_s[key * d + j] = vv;
        }
        __syncthreads();

#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            const int row = warp * kRowsPerWarp + r;
            if (row >= rows_here) continue;                  // uniform within the warp
            const int q_pos = first_pos + row;
            const int kp = k0 + lane;
            const float* q_row = q_s + row * d;
            const float* k_row = k_s + lane * (d + 1);
            float score = 0.0f;
            for (int j = 0; j < d; ++j) score = fmaf(q_row[j], k_row[j], score);
            score *= scale;
            bool visible = kp <= q_pos;
            if (window > 0) visible = visible && (kp > q_pos - window);
            if (!visible) score = -INFINITY;
            const float new_max = fmaxf(row_max[r], warp_max(score));
            if (new_max == -INFINITY) continue;              // nothing visible so far
            const float correction = expf(row_max[r] - new_max);   // exp(-inf) = 0 on the first tile
            const float p = visible ? expf(score - new_max) : 0.0f;
            row_sum[r] = row_sum[r] * correction + warp_sum(p);
            row_max[r] = new_max;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[r][i] *= correction;
            for (int key = 0; key < kKeyTile; ++key) {
                const float pk = __shfl_sync(0xffffffffu, p, key);
                const float* v_row = v_s + key * d;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int j = lane + 32 * i;
                    if (j < d) acc[r][i] = fmaf(pk, v_row[j], acc[r][i]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const int row = warp * kRowsPerWarp + r;
        if (row >= rows_here) continue;
        const float inv = row_sum[r] > 0.0f ? 1.0f / row_sum[r] : 0.0f;
        T* dst = out + ((size_t)(q_begin + tile_first + row) * nq + head) * d;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int j = lane + 32 * i;
            if (j < d) dst[j] = from_float<T>(acc[r][i] * inv);
        }
    }
}

template <typename T, int DPL>
int launch_generic(const void* q, const void* k_pages, const void* v_pages, void* out,
                   const int* query_start, const int* seq_lens, const int* block_table,
                   int num_requests, int num_tokens, int max_pages, int nq, int nkv, int d,
                   int page_size, float scale, int window, cudaStream_t stream) {
    auto kernel = paged_attention_generic_kernel<T, DPL>;
    const size_t smem = sizeof(float) * ((size_t)kQueryTile * d + (size_t)kKeyTile * (d + 1) + (size_t)kKeyTile * d);
    if (smem > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("paged_attention_generic", cudaGetErrorString(status));
    }
    dim3 grid(num_tokens / kQueryTile + num_requests, nq);
    kernel<<<grid, kWarps * 32, smem, stream>>>(
        (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, query_start, seq_lens,
        block_table, num_requests, max_pages, nq, nkv, d, page_size, scale, window);
    return check_launch("paged_attention_generic");
}

template <typename T>
int dispatch_generic(const void* q, const void* k_pages, const void* v_pages, void* out,
                     const int* query_start, const int* seq_lens, const int* block_table,
                     int num_requests, int num_tokens, int max_pages, int nq, int nkv, int d,
                     int page_size, float scale, int window, cudaStream_t stream) {
#define B200_CASE(DPL)                                                                            \
    if (d <= 32 * DPL)                                                                            \
        return launch_generic<T, DPL>(q, k_pages, v_pages, out, query_start, seq_lens, block_table, \
                                      num_requests, num_tokens, max_pages, nq, nkv, d, page_size,  \
                                      scale, window, stream);
    B200_CASE(1) B200_CASE(2) B200_CASE(4) B200_CASE(8) B200_CASE(16)
#undef B200_CASE
    return fail("paged_attention_generic", "head_dim above 512 is not built");
}

}  // namespace b200

// window <= 0: every earlier key is visible.  dtype: 0 = float32, 1 = bfloat16.
B200_EXPORT int b200_paged_attention_generic(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
    const int* seq_lens, const int* block_table, int num_requests, int num_tokens, int max_pages,
    int nq, int nkv, int d, int page_size, float scale, int window, int dtype, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens == 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv) return fail("paged_attention_generic", "query heads must be a multiple of key/value heads");
    if (nq > 65535) return fail("paged_attention_generic", "more than 65535 query heads");
    if (d <= 0 || page_size <= 0 || max_pages <= 0) return fail("paged_attention_generic", "sizes must be positive");
    if (dtype == 0)
        return dispatch_generic<float>(q, k_pages, v_pages, out, query_start, seq_lens, block_table,
                                       num_requests, num_tokens, max_pages, nq, nkv, d, page_size, scale, window, stream);
    if (dtype == 1)
        return dispatch_generic<__nv_bfloat16>(q, k_pages, v_pages, out, query_start, seq_lens, block_table,
                                               num_requests, num_tokens, max_pages, nq, nkv, d, page_size, scale, window, stream);
    return fail("paged_attention_generic", "dtype must be 0 (float32) or 1 (bfloat16)");
}

// Exported launchers of the bfloat16 tensor-core attention kernels; the kernels
// themselves are in attention_bf16_kernels.cuh.
#include "attention_bf16_kernels.cuh"
#include "attention_tc.cuh"
#include "decode_attention_tma.cuh"
#include "tensor_map.cuh"

// Returns 1 if head_dim / head counts are ones these kernels are built for.
B200_EXPORT int b200_attention_bf16_supports(int nq, int nkv, int d) {
    return (d == 64 || d == 128 || d == 256) && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16 && nq <= 65535
               ? 1 : 0;
}

// Decode batches: exactly one query token per request.  With splits > 1,
// partial_o holds [requests * nq * splits * d] floats and partial_ml
// [requests * nq * splits * 2] floats of scratch.
B200_EXPORT int b200_decode_attention_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, float* partial_o,
    float* partial_ml, const int* seq_lens, const int* block_table, int num_requests, int max_pages,
    int nq, int nkv, int d, int page_size, float scale, int window, int splits, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0) return 0;
    if (!b200_attention_bf16_supports(nq, nkv, d)) return fail("decode_attention", "shape not built");
    if (splits < 1 || nkv > 65535 || num_requests > 65535) return fail("decode_attention", "grid out of range");
    if (splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("decode_attention", "scratch for the splits is missing");
#define B200_CASE(D)                                                                                   \
    if (d == D)                                                                                        \
        return launch_decode<D>(q, k_pages, v_pages, out, partial_o, partial_ml, seq_lens, block_table, \
                                num_requests, max_pages, nq, nkv, page_size, scale, window, splits, stream);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("decode_attention", "head_dim not built");
}

// 1 if the decode kernel with tensor copies takes this shape (pages of 8, 16, 32, ... keys).
B200_EXPORT int b200_decode_attention_tma_supports(int nq, int nkv, int d, int page_size) {
    return b200_attention_bf16_supports(nq, nkv, d) && page_size >= 8 && (page_size & (page_size - 1)) == 0 ? 1 : 0;
}

static int* attention_error_flag();

// The same contract as b200_decode_attention_bf16; num_pages: pages in k_pages / v_pages.
B200_EXPORT int b200_decode_attention_tma_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, float* partial_o,
    float* partial_ml, const int* seq_lens, const int* block_table, int num_requests, int max_pages,
    int nq, int nkv, int d, int page_size, int num_pages, float scale, int window, int splits,
    cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0) return 0;
    if (!b200_decode_attention_tma_supports(nq, nkv, d, page_size)) return fail("decode_attention", "shape not built");
    if (splits < 1 || nkv > 65535 || num_requests > 65535) return fail("decode_attention", "grid out of range");
    if (splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("decode_attention", "scratch for the splits is missing");
    int* error_flag = attention_error_flag();
    if (error_flag == nullptr) return fail("decode_attention", "no error flag");
    const int copy_rows = page_size < kKeys ? page_size : kKeys;
    CUtensorMap map_k, map_v;
    if (!tensor_map_for(k_pages, num_pages * nkv * page_size, d, copy_rows, &map_k) ||
        !tensor_map_for(v_pages, num_pages * nkv * page_size, d, copy_rows, &map_v))
        return fail("decode_attention", "could not encode a tensor map");
#define B200_CASE(D)                                                                                        \
    if (d == D)                                                                                             \
        return launch_decode_tma<D, false>(map_k, map_v, q, out, partial_o, partial_ml, seq_lens,          \
                                           block_table, num_requests, max_pages, nq, nkv, page_size, scale, \
                                           window, splits, error_flag, stream);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("decode_attention", "head_dim not built");
}

// 1 if the decode kernel that also normalises and rotates the heads and stores the new key and value takes the shape.
B200_EXPORT int b200_decode_attention_fused_supports(int nq, int nkv, int d, int rotary_dim, int page_size) {
    return d == 128 && rotary_dim == d && b200_decode_attention_tma_supports(nq, nkv, d, page_size) ? 1 : 0;
}

// One decode step's attention from the packed projection qkv [T, (nq + 2 nkv) d], one token per request:
// what b200_head_norm_rope_cache (rope_cache.cu) followed by b200_decode_attention_tma_bf16 does.
B200_EXPORT int b200_decode_attention_fused_bf16(
    const void* qkv, const int* positions, const int* slots, const float* q_weight, const float* k_weight,
    const float* inv_freq, float eps, void* k_pages, void* v_pages, void* out, float* partial_o,
    float* partial_ml, const int* seq_lens, const int* block_table, int num_requests, int max_pages, int nq,
    int nkv, int d, int page_size, int num_pages, float scale, int window, int splits, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0) return 0;
    if (!b200_decode_attention_fused_supports(nq, nkv, d, d, page_size)) return fail("decode_attention", "shape not built");
    if (splits < 1 || nkv > 65535 || num_requests > 65535) return fail("decode_attention", "grid out of range");
    if (splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("decode_attention", "scratch for the splits is missing");
    int* error_flag = attention_error_flag();
    if (error_flag == nullptr) return fail("decode_attention", "no error flag");
    const int copy_rows = page_size < kKeys ? page_size : kKeys;
    CUtensorMap map_k, map_v;
    if (!tensor_map_for(k_pages, num_pages * nkv * page_size, d, copy_rows, &map_k) ||
        !tensor_map_for(v_pages, num_pages * nkv * page_size, d, copy_rows, &map_v))
        return fail("decode_attention", "could not encode a tensor map");
    DecodeRope rope;
    rope.positions = positions;
    rope.slots = slots;
    rope.q_weight = q_weight;
    rope.k_weight = k_weight;
    rope.inv_freq = inv_freq;
    rope.k_pages = (bf16*)k_pages;
    rope.v_pages = (bf16*)v_pages;
    rope.eps = eps;
    return launch_decode_tma<128, true>(map_k, map_v, qkv, out, partial_o, partial_ml, seq_lens, block_table,
                                        num_requests, max_pages, nq, nkv, page_size, scale, window, splits,
                                        error_flag, stream, rope);
}

B200_EXPORT int b200_prefill_attention_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
    const int* seq_lens, const int* block_table, int num_requests, int num_tokens, int max_pages, int nq,
    int nkv, int d, int page_size, float scale, int window, int token_offset, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens - token_offset <= 0) return 0;
    if (token_offset < 0) return fail("prefill_attention", "negative token offset");
    if (!b200_attention_bf16_supports(nq, nkv, d)) return fail("prefill_attention", "shape not built");
#define B200_CASE(D)                                                                                     \
    if (d == D)                                                                                          \
        return launch_prefill<D>(q, k_pages, v_pages, out, query_start, seq_lens, block_table,           \
                                 num_requests, num_tokens, max_pages, nq, nkv, page_size, scale, window, \
                                 token_offset, stream);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("prefill_attention", "head_dim not built");
}

namespace b200 {
// Set by a kernel whose bounded wait ran out (0 = never); read and cleared by b200_attention_error().
__device__ int g_attention_error;
}  // namespace b200

// Device address of the error flag (per device of the calling thread), or null.
static int* attention_error_flag() {
    static int* address[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (address[device] == nullptr) {
        void* found = nullptr;
        if (cudaGetSymbolAddress(&found, b200::g_attention_error) != cudaSuccess) return nullptr;
        address[device] = static_cast<int*>(found);
    }
    return address[device];
}

// Device address of the error word (for a reader that copies it with other results), or null.
B200_EXPORT void* b200_attention_error_address() { return attention_error_flag(); }

B200_EXPORT int b200_attention_error() {
    int code = 0;
    if (cudaMemcpyFromSymbol(&code, b200::g_attention_error, sizeof(int)) != cudaSuccess) return -1;
    if (code != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(b200::g_attention_error, &zero, sizeof(int));
    }
    return code;
}

// 1 if the tcgen05 kernel takes this shape: head size 128, pages of 8, 16, 32, 64 or 128 keys.
B200_EXPORT int b200_prefill_attention_tc_supports(int nq, int nkv, int d, int page_size) {
    return d == 128 && nkv > 0 && nq % nkv == 0 && nq <= 65535 && page_size >= 8 && page_size <= 128 &&
                   (page_size & (page_size - 1)) == 0
               ? 1 : 0;
}

// Number of SMs of the calling thread's device, 0 if it cannot be read.
B200_EXPORT int b200_sm_count() { return b200::sm_count(); }

// Host-only check that maps handed out by the tensor-map cache stay valid when the cache is
// emptied (see tensor_map.cuh); buffer: `bytes` of device memory whose addresses are encoded
// and never read.  0 = all copies agree.
B200_EXPORT int b200_tensor_map_cache_self_check(const void* buffer, long long bytes, int count) {
    return b200::tensor_map_cache_self_check(buffer, (size_t)bytes, count);
}

// Over how many blocks the tensor-memory kernel divides the keys of a row block for a launch of
// num_tokens tokens of num_requests requests (1: not at all).  The caller provides
// partial_o [rows of q * nq * splits, 128] and partial_ml [rows of q * nq * splits, 2] floats.
B200_EXPORT int b200_prefill_attention_tc_splits(int num_tokens, int num_requests, int nq, int max_seq_len) {
    const int sms = b200::sm_count();
    const long long blocks = (long long)(num_tokens / b200::kAtBlockRows + num_requests) * nq;
    if (sms <= 0 || blocks <= 0 || blocks * 2 > sms) return 1;          // half the SMs busy: leave it
    int splits = (int)(sms / blocks);
    // Sixteen tiles of keys a block at least: 512 tokens over 512 keys took 25 us in two shares
    // against 15 us whole, 512 over 8192 keys 75 against 156 us, 128 over 16384 keys 48 against 288.
    const int by_keys = max_seq_len / 1024;
    if (splits > by_keys) splits = by_keys;
    if (splits > 8) splits = 8;
    return splits < 2 ? 1 : splits;
}

// The tensor-memory kernel for portions of prompts.  num_pages: pages in k_pages / v_pages.
// q and out hold num_tokens rows and query_start rows of them; the num_requests requests
// given here begin at row token_offset (what lies ahead of it is another launch's).
B200_EXPORT int b200_prefill_attention_tc_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
    const int* seq_lens, const int* block_table, int num_requests, int num_tokens, int max_pages, int nq,
    int nkv, int d, int page_size, int num_pages, float scale, int window, int token_offset, int key_splits,
    float* partial_o, float* partial_ml, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens - token_offset <= 0) return 0;
    if (token_offset < 0) return fail("prefill_attention_tc", "negative token offset");
    if (key_splits < 1 || key_splits > 16) return fail("prefill_attention_tc", "key_splits out of range");
    if (key_splits > 1 && (partial_o == nullptr || partial_ml == nullptr))
        return fail("prefill_attention_tc", "scratch for the splits is missing");
    if (!b200_prefill_attention_tc_supports(nq, nkv, d, page_size)) return fail("prefill_attention_tc", "shape not built");
    int* error_flag = attention_error_flag();
    if (error_flag == nullptr) return fail("prefill_attention_tc", "no error flag");
    const int copy_rows = page_size < kAtKeys ? page_size : kAtKeys;            // a page, or the part of it in one tile
    CUtensorMap map_q, map_k, map_v;
    if (!tensor_map_for(q, num_tokens, nq * d, kAtRows, &map_q) ||             // one group of rows per copy
        !tensor_map_for(k_pages, num_pages * nkv * page_size, d, copy_rows, &map_k) ||
        !tensor_map_for(v_pages, num_pages * nkv * page_size, d, copy_rows, &map_v))
        return fail("prefill_attention_tc", "could not encode a tensor map");
    cudaError_t status = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtSmem);
    if (status != cudaSuccess) return fail("prefill_attention_tc", cudaGetErrorString(status));
    const int blocks = (num_tokens - token_offset) / kAtBlockRows + num_requests;
    if (blocks > 65535) return fail("prefill_attention_tc", "too many tokens for one launch");
    dim3 grid(nq, blocks, key_splits);
    launch_overlapped(prefill_attention_tc_kernel, grid, dim3(kAtThreads), kAtSmem, stream,
        map_q, map_k, map_v, (__nv_bfloat16*)out, query_start, seq_lens, block_table, num_requests, max_pages,
        nq, nkv, page_size, scale * kLog2e, window, token_offset, key_splits, partial_o, partial_ml, error_flag);
    if (int rc = check_launch("prefill_attention_tc")) return rc;
    if (key_splits > 1) {
        const size_t first = (size_t)token_offset * nq;                 // (row of q, head) pairs ahead of this launch
        launch_overlapped(merge_splits_kernel<kAtD>, (num_tokens - token_offset) * nq, 128, 0, stream,
                          (const float*)(partial_o + first * key_splits * kAtD),
                          (const float*)(partial_ml + first * key_splits * 2),
                          (bf16*)out + first * kAtD, key_splits);
        return check_launch("merge_splits");
    }
    return 0;
}

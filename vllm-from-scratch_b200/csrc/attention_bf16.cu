// Exported launchers of the bfloat16 tensor-core attention kernels; the kernels
// themselves are in attention_bf16_kernels.cuh.
#include "attention_bf16_kernels.cuh"

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

B200_EXPORT int b200_prefill_attention_bf16(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* query_start,
    const int* seq_lens, const int* block_table, int num_requests, int num_tokens, int max_pages, int nq,
    int nkv, int d, int page_size, float scale, int window, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0 || num_tokens == 0) return 0;
    if (!b200_attention_bf16_supports(nq, nkv, d)) return fail("prefill_attention", "shape not built");
#define B200_CASE(D)                                                                                     \
    if (d == D)                                                                                          \
        return launch_prefill<D>(q, k_pages, v_pages, out, query_start, seq_lens, block_table,           \
                                 num_requests, num_tokens, max_pages, nq, nkv, page_size, scale, window, stream);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("prefill_attention", "head_dim not built");
}

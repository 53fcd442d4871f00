// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (tutu04538/vllm-from-scratch):
// it exists for users of this library, not for parity.
//
// Who needs it: a host program that handed the whole device to another allocator
// at start-up, so that cudaMalloc fails or is forbidden by policy; a plug-in that
// is given raw device pointers and a stream by the framework around it and must
// leave that framework's allocator alone; a latency-critical loop in which the
// implicit synchronisation of an allocation is not acceptable.  The ordinary
// split-key decode attention (b200_decode_attention_bf16) needs scratch memory for
// the partial results of the splits, which its caller has to allocate.  This
// variant keeps that scratch in a fixed array inside the library instead, so the
// caller passes inputs and outputs only.
//
// Limits and rules:
//   * num_requests * nq * splits <= B200_STATIC_MAX_PARTIAL_ROWS (8192) and
//     d <= B200_STATIC_MAX_HEAD_DIM (256); anything larger is refused with an
//     error, never truncated.  The array takes about 8.4 MB of every GPU on which
//     the library is used, from the first call until the process exits.
//   * The first call on a device looks up the array's device address (once per
//     device, with that device current).  Make that first call before any stream
//     capture begins.
//   * The function calls no cudaMalloc, cudaFree or any allocating routine.
//   * All calls share the one array, and it keeps what the last call left in it.
//     Every slot a call reads is written earlier in that same call, so nothing
//     needs clearing; but two calls that overlap on the GPU (different streams, or
//     another process thread) race on the array.  Run them one after the other.
//
// Arguments are those of b200_decode_attention_bf16 without the two scratch
// pointers: bfloat16 q [requests, nq * d] (one query token per request), key and
// value pages [pages, nkv, page_size, d], out [requests, nq * d], int32 seq_lens
// [requests], int32 block_table [requests, max_pages]; window <= 0 means all keys;
// splits >= 1 blocks share the keys of one (request, key/value head).
// Returns 0, or a negative value after storing a message for b200_last_error().
#pragma once

#include <cuda_runtime.h>

#define B200_STATIC_MAX_PARTIAL_ROWS 8192
#define B200_STATIC_MAX_HEAD_DIM 256

#ifdef __cplusplus
extern "C" {
#endif

int b200_decode_attention_bf16_static(const void* q, const void* k_pages, const void* v_pages, void* out,
                                      const int* seq_lens, const int* block_table, int num_requests,
                                      int max_pages, int nq, int nkv, int d, int page_size, float scale,
                                      int window, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

// Split-key decode attention whose scratch memory is a fixed array in this
// library: see decode_attention_static.h for who needs it and for its rules.
#include "decode_attention_static.h"

#include "attention_bf16_kernels.cuh"

namespace {

// Partial outputs [rows][d] followed by partial (maximum, sum) pairs [rows][2].
constexpr size_t kPartialFloats =
    (size_t)B200_STATIC_MAX_PARTIAL_ROWS * (B200_STATIC_MAX_HEAD_DIM + 2);
static __device__ __align__(256) float g_partials[kPartialFloats];

constexpr int kMaxDevices = 64;
float* g_partials_address[kMaxDevices] = {};

// In host code `g_partials` is only a handle for the runtime, not a device
// address: the address is asked for once per device, with that device current.
int partials_on_current_device(float** address) {
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return b200::fail("decode_attention_static", cudaGetErrorString(status));
    if (device < 0 || device >= kMaxDevices)
        return b200::fail("decode_attention_static", "device ordinal out of range");
    if (g_partials_address[device] == nullptr) {
        void* found = nullptr;
        status = cudaGetSymbolAddress(&found, g_partials);
        if (status != cudaSuccess) return b200::fail("decode_attention_static", cudaGetErrorString(status));
        g_partials_address[device] = static_cast<float*>(found);
    }
    *address = g_partials_address[device];
    return 0;
}

}  // namespace

B200_EXPORT int b200_decode_attention_bf16_static(
    const void* q, const void* k_pages, const void* v_pages, void* out, const int* seq_lens,
    const int* block_table, int num_requests, int max_pages, int nq, int nkv, int d, int page_size,
    float scale, int window, int splits, cudaStream_t stream) {
    using namespace b200;
    if (num_requests == 0) return 0;
    const bool shape_ok = (d == 64 || d == 128 || d == 256) && nkv > 0 && nq % nkv == 0 &&
                          nq / nkv <= 16 && nq <= 65535;
    if (!shape_ok) return fail("decode_attention_static", "shape not built");
    if (splits < 1 || nkv > 65535 || num_requests > 65535 || num_requests < 0)
        return fail("decode_attention_static", "grid out of range");
    if (d > B200_STATIC_MAX_HEAD_DIM)
        return fail("decode_attention_static", "head_dim exceeds B200_STATIC_MAX_HEAD_DIM");
    const long long rows = (long long)num_requests * nq * splits;
    if (rows > B200_STATIC_MAX_PARTIAL_ROWS)
        return fail("decode_attention_static",
                    "num_requests * nq * splits exceeds B200_STATIC_MAX_PARTIAL_ROWS (8192)");
    float* partials = nullptr;
    if (int rc = partials_on_current_device(&partials)) return rc;
    float* partial_o = partials;
    float* partial_ml = partials + (size_t)rows * d;
#define B200_CASE(D)                                                                                   \
    if (d == D)                                                                                        \
        return launch_decode<D>(q, k_pages, v_pages, out, partial_o, partial_ml, seq_lens, block_table, \
                                num_requests, max_pages, nq, nkv, page_size, scale, window, splits, stream);
    B200_CASE(64) B200_CASE(128) B200_CASE(256)
#undef B200_CASE
    return fail("decode_attention_static", "head_dim not built");
}

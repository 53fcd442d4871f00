// bfloat16 matrix products for few rows: y[M, N] = x[M, K] . w[N, K]^T with
// M <= 16, float32 accumulation, output bfloat16 or float32.
//
// With so few rows the product is a stream of the weight matrix through the SMs:
// every weight is used once, so the kernel is built to keep many 16-byte loads in
// flight and nothing else.  One block owns 8 (or 2 x 8) weight rows; its warps (4 to
// 16, more the fewer blocks the product has) split K in interleaved blocks of 32, so
// that together they read long contiguous pieces of each row per round.  The products run on the tensor cores
// (m16n8k16, rows of the fragment = the tokens, columns = the 8 weight rows) with
// the k index permuted the same way in both operands: a thread's 16-byte load of
// a weight row and of a token row are the fragments of two k-steps as they are, no
// shuffles.  The warps' partial sums are added in a fixed order, so a token's result
// does not depend on how many other tokens share the launch.
//
// The gated variant computes silu(x w_gate^T) * (x w_up^T) for the two row blocks
// [0, I) and [I, 2I) of one matrix (minivllm/models/qwen3.py:44-65 as one kernel).
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "async_copy.cuh"

namespace b200 {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                             unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const bf16* p) {
    // weights are read once: do not keep them in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <typename T> __device__ __forceinline__ void store_pair(T* p, float a, float b);
template <> __device__ __forceinline__ void store_pair<bf16>(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <> __device__ __forceinline__ void store_pair<float>(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <typename T> __device__ __forceinline__ void store_one(T* p, float a) { *p = from_float<T>(a); }

}  // namespace b200
#include "slab_gemm.cuh"
namespace b200 {

constexpr int kSkinnyMaxWarps = 16;

// TILES: weight-row blocks of 8 per CTA.  GATED: TILES must be 2; block 0 = gate rows, block 1 = up rows.
// The block's warps (blockDim.x / 32, at most 16) split K; each keeps UNROLL blocks of 32 in flight.
template <int TILES, bool GATED, typename OutT, int UNROLL>
__global__ void __launch_bounds__(kSkinnyMaxWarps * 32) skinny_gemm_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ w, OutT* __restrict__ y, int M, int N, int K,
    int up_offset) {
    __shared__ float partial[kSkinnyMaxWarps][TILES][32][4];
    overlap_trigger();
    const int kSkinnyWarps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * (GATED ? 8 : 8 * TILES);

    const bf16* w_row[TILES];
    bool w_ok[TILES];
#pragma unroll
    for (int i = 0; i < TILES; ++i) {
        const int n = GATED ? (n0 + g + i * up_offset) : (n0 + i * 8 + g);
        w_ok[i] = GATED ? (n0 + g < N) : (n < N);
        w_row[i] = w + (size_t)(w_ok[i] ? n : 0) * K + 8 * t;
    }
    const bool x_lo = g < M, x_hi = g + 8 < M;
    const bf16* x_row_lo = x + (size_t)(x_lo ? g : 0) * K + 8 * t;
    const bf16* x_row_hi = x + (size_t)(x_hi ? g + 8 : 0) * K + 8 * t;

    float acc[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

    const int blocks = K >> 5;                          // K is a multiple of 32
    constexpr int kUnroll = UNROLL;
    overlap_wait();                                     // the token rows come from the kernel before this one
    const uint4 zero = make_uint4(0, 0, 0, 0);
    int j = warp;
    for (; j + (kUnroll - 1) * kSkinnyWarps < blocks; j += kUnroll * kSkinnyWarps) {
        uint4 wv[kUnroll][TILES], xl[kUnroll], xh[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int off = (j + u * kSkinnyWarps) << 5;
#pragma unroll
            for (int i = 0; i < TILES; ++i) wv[u][i] = w_ok[i] ? load_stream(w_row[i] + off) : zero;
            xl[u] = x_lo ? *reinterpret_cast<const uint4*>(x_row_lo + off) : zero;
            xh[u] = x_hi ? *reinterpret_cast<const uint4*>(x_row_hi + off) : zero;
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int i = 0; i < TILES; ++i) {
                mma_m16n8k16(acc[i], xl[u].x, xh[u].x, xl[u].y, xh[u].y, wv[u][i].x, wv[u][i].y);
                mma_m16n8k16(acc[i], xl[u].z, xh[u].z, xl[u].w, xh[u].w, wv[u][i].z, wv[u][i].w);
            }
    }
    for (; j < blocks; j += kSkinnyWarps) {
        const int off = j << 5;
        const uint4 xl = x_lo ? *reinterpret_cast<const uint4*>(x_row_lo + off) : zero;
        const uint4 xh = x_hi ? *reinterpret_cast<const uint4*>(x_row_hi + off) : zero;
#pragma unroll
        for (int i = 0; i < TILES; ++i) {
            const uint4 wv = w_ok[i] ? load_stream(w_row[i] + off) : zero;
            mma_m16n8k16(acc[i], xl.x, xh.x, xl.y, xh.y, wv.x, wv.y);
            mma_m16n8k16(acc[i], xl.z, xh.z, xl.w, xh.w, wv.z, wv.w);
        }
    }

#pragma unroll
    for (int i = 0; i < TILES; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) partial[warp][i][lane][e] = acc[i][e];
    __syncthreads();
    if (warp != 0) return;
    float total[TILES][4];
#pragma unroll
    for (int i = 0; i < TILES; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float s = partial[0][i][lane][e];
            for (int wi = 1; wi < kSkinnyWarps; ++wi) s += partial[wi][i][lane][e];
            total[i][e] = s;
        }
    // accumulator layout: c0, c1 = (token g, weight rows 2t, 2t+1), c2, c3 = (token g + 8, same rows)
    if (GATED) {
        const int n = n0 + 2 * t;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int token = g + half * 8;
            if (token >= M) continue;
            const float g0 = total[0][half * 2], g1 = total[0][half * 2 + 1];
            const float u0 = total[1][half * 2], u1 = total[1][half * 2 + 1];
            const float r0 = g0 / (1.0f + expf(-g0)) * u0, r1 = g1 / (1.0f + expf(-g1)) * u1;
            OutT* dst = y + (size_t)token * N + n;
            if (n + 1 < N && (N & 1) == 0) store_pair<OutT>(dst, r0, r1);
            else {
                if (n < N) store_one<OutT>(dst, r0);
                if (n + 1 < N) store_one<OutT>(dst + 1, r1);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < TILES; ++i) {
            const int n = n0 + i * 8 + 2 * t;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int token = g + half * 8;
                if (token >= M) continue;
                OutT* dst = y + (size_t)token * N + n;
                if (n + 1 < N && (N & 1) == 0) store_pair<OutT>(dst, total[i][half * 2], total[i][half * 2 + 1]);
                else {
                    if (n < N) store_one<OutT>(dst, total[i][half * 2]);
                    if (n + 1 < N) store_one<OutT>(dst + 1, total[i][half * 2 + 1]);
                }
            }
        }
    }
}

template <typename OutT>
int launch_skinny(const bf16* x, const bf16* w, OutT* y, int M, int N, int K, int gated_inter,
                  cudaStream_t stream) {
    // The GPU should hold a few thousand warps, each with all of its loads in flight:
    // the fewer blocks a product has, the more warps split K inside each block.
    const int k_blocks = K >> 5;
    const bool two_tiles = gated_inter > 0 || N >= sm_count() * 4 * 16;
    const int ctas = gated_inter > 0 ? (gated_inter + 7) / 8 : two_tiles ? (N + 15) / 16 : (N + 7) / 8;
    const int wanted = 6144 / (ctas * (two_tiles ? 2 : 1));
    int warps = 4;
    while (warps * 2 <= wanted && warps < kSkinnyMaxWarps) warps *= 2;
    while (warps > 1 && warps > k_blocks) warps /= 2;
    const int threads = warps * 32;
    if (gated_inter > 0) {
        launch_overlapped(skinny_gemm_kernel<2, true, OutT, 4>, ctas, threads, 0, stream, x, w, y, M, gated_inter, K, gated_inter);
    } else if (two_tiles) {
        launch_overlapped(skinny_gemm_kernel<2, false, OutT, 4>, ctas, threads, 0, stream, x, w, y, M, N, K, 0);
    } else {
        launch_overlapped(skinny_gemm_kernel<1, false, OutT, 8>, ctas, threads, 0, stream, x, w, y, M, N, K, 0);
    }
    return check_launch("skinny_gemm");
}

// Set by a kernel whose bounded wait ran out (0 = never).  Read and cleared by
// b200_stream_gemm_error().
__device__ int g_stream_error;

// Device address of the error word, per device of the calling thread, or null.
inline int* stream_error_flag() {
    static int* address[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (address[device] == nullptr) {
        void* found = nullptr;
        if (cudaGetSymbolAddress(&found, g_stream_error) != cudaSuccess) return nullptr;
        address[device] = static_cast<int*>(found);
    }
    return address[device];
}

// 1 = launched, 0 = not a shape for the kernel with resident weight rows, < 0 = error.
// gated_inter > 0: w is [2 * gated_inter, K], the result [M, gated_inter].
template <typename OutT>
int launch_slab(const bf16* x, const bf16* w, OutT* y, int M, int N, int K, int gated_inter, cudaStream_t stream,
                const SlabNorm& norm = SlabNorm{}) {
    const bool gated = gated_inter > 0;
    if (M > 16 || K % 128 != 0 || slab_smem_bytes(K, gated) > 200 * 1024) return 0;
    int* error_flag = stream_error_flag();
    if (error_flag == nullptr) return fail("slab_gemm", "no error flag");
    const size_t smem = slab_smem_bytes(K, gated);
    const int rows = gated ? gated_inter : N;
    const int blocks = (rows + kSlabRows - 1) / kSlabRows, threads = kSlabWarps * 32;
    const bool wide = M > 8;
    // More fragments of the token rows in flight (the sums are formed in the same order either
    // way): for one or two token rows, where a decode step took 1.193 against 1.213 ms with it (at 8
    // rows 1.504 against 1.499), in the plain form where two blocks of such rows fill an SM's shared
    // memory, in the gated form always.
    const bool deep = M <= 2 && (gated || K >= 4096);
    auto launch = [&](auto kernel, bool* configured) {
        if (!*configured) {
            cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (status != cudaSuccess) return fail("slab_gemm", cudaGetErrorString(status));
            *configured = true;
        }
        launch_overlapped(kernel, blocks, threads, smem, stream, x, w, y, M, rows, K, error_flag, norm);
        return 0;
    };
    static bool configured[4 * 7] = {};
    const int halves = (norm.squares_in != nullptr ? 1 : 0) | (norm.residual != nullptr ? 2 : 0);
    int rc;
    // (the halves of a norm are for bfloat16 results only: the float32 result has the plain form alone)
    constexpr int kOne = std::is_same<OutT, bf16>::value ? 1 : 0, kTwo = kOne * 2, kBoth = kOne * 3;
    if (halves != 0 && kOne == 0) return fail("slab_gemm", "the halves of a norm need a bfloat16 result");
#define B200_SLAB(G, W, D, slot)                                                                                   \
    rc = halves == 0   ? launch(slab_gemm_kernel<OutT, G, W, D, 0>, configured + slot)                             \
         : halves == 1 ? launch(slab_gemm_kernel<OutT, G, W, D, kOne>, configured + 7 + slot)                      \
         : halves == 2 ? launch(slab_gemm_kernel<OutT, G, W, D, kTwo>, configured + 14 + slot)                     \
                       : launch(slab_gemm_kernel<OutT, G, W, D, kBoth>, configured + 21 + slot)
    // (a gated product never carries the sum: two instantiations each)
#define B200_SLAB_GATED(W, D, slot)                                                                                \
    rc = halves == 0 ? launch(slab_gemm_kernel<OutT, true, W, D, 0>, configured + slot)                            \
                     : launch(slab_gemm_kernel<OutT, true, W, D, kOne>, configured + 7 + slot)
    if (gated && (halves & 2)) return fail("slab_gemm", "a gated product cannot add into the residual");
    if (gated && wide) B200_SLAB_GATED(true, false, 0);
    else if (gated && deep) B200_SLAB_GATED(false, true, 1);
    else if (gated) B200_SLAB_GATED(false, false, 6);
    else if (wide && deep) B200_SLAB(false, true, true, 2);
    else if (wide) B200_SLAB(false, true, false, 3);
    else if (deep) B200_SLAB(false, false, true, 4);
    else B200_SLAB(false, false, false, 5);
#undef B200_SLAB
#undef B200_SLAB_GATED
    if (rc != 0) return -1;
    return check_launch("slab_gemm") == 0 ? 1 : -1;
}

}  // namespace b200

// 0, or the code a kernel left when one of its bounded waits ran out (41, 42: a block of the
// resident-rows kernel waited for its weight rows).
// Synchronises with the device and clears the code.
// Device address of the error word (for a reader that copies it with other results), or null.
B200_EXPORT void* b200_stream_gemm_error_address() { return b200::stream_error_flag(); }

B200_EXPORT int b200_stream_gemm_error() {
    int code = 0;
    if (cudaMemcpyFromSymbol(&code, b200::g_stream_error, sizeof(int)) != cudaSuccess) return -1;
    if (code != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(b200::g_stream_error, &zero, sizeof(int));
    }
    return code;
}

#include "tensor_map.cuh"
#include "tc_gemm.cuh"
namespace b200 {

template <int BN>
int launch_tc_gated_gemm(const bf16* x, const bf16* w, bf16* y, int M, int inter, int K, cudaStream_t stream) {
    int* error_flag = stream_error_flag();
    if (error_flag == nullptr) return fail("tc_gated_gemm", "no error flag");
    CUtensorMap map_x, map_w;
    if (!tensor_map_for(x, M, K, kTgRows, &map_x) || !tensor_map_for(w, 2 * inter, K, BN / 2, &map_w))
        return fail("tc_gated_gemm", "could not encode a tensor map");
    auto kernel = tc_gated_gemm_kernel<BN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcGemmShape<BN>::kSmem);
        if (status != cudaSuccess) return fail("tc_gated_gemm", cudaGetErrorString(status));
        configured = true;
    }
    const int tiles = ((M + kTgRows - 1) / kTgRows) * (inter / (BN / 2));
    const int blocks = tiles < sm_count() ? tiles : sm_count();
    launch_overlapped(kernel, blocks, kTgThreads, TcGemmShape<BN>::kSmem, stream, map_x, map_w, y, M, inter, K, error_flag);
    return check_launch("tc_gated_gemm");
}

// Weight rows per tile (gate and up together) that the tensor-memory gated product would use, 0 if it
// does not take the shape: the tile with the fewer rounds over the SMs, weighted by its width.
inline int tc_gated_gemm_tile(int M, int inter, int K) {
    if (M < 1 || K < kTgK || K % kTgK != 0) return 0;
    const int sms = sm_count();
    if (sms <= 0) return 0;
    int best = 0;
    long long best_cost = 0;
    const int candidates[2] = {256, 192};
    for (int i = 0; i < 2; ++i) {
        const int tile = candidates[i];
        if (inter % (tile / 2) != 0) continue;
        const long long tiles = (long long)((M + kTgRows - 1) / kTgRows) * (inter / (tile / 2));
        const long long cost = ((tiles + sms - 1) / sms) * tile;
        if (best == 0 || cost < best_cost) {
            best = tile;
            best_cost = cost;
        }
    }
    return best;
}

}  // namespace b200

// Weight rows per tile of the tensor-memory gated product (tc_gemm.cuh) for M token rows and a
// [2 * inter, K] matrix, or 0 if the kernel does not take the shape.
B200_EXPORT int b200_tc_gated_gemm_tile(int M, int inter, int K) { return b200::tc_gated_gemm_tile(M, inter, K); }

// y[M, inter] = silu(x w[:inter]^T) * (x w[inter:]^T), bfloat16, on the 5th-generation tensor cores.
B200_EXPORT int b200_tc_gated_gemm_bf16(const void* x, const void* w, void* y, int M, int inter, int K, cudaStream_t stream) {
    using namespace b200;
    if (M == 0 || inter == 0) return 0;
    const int tile = tc_gated_gemm_tile(M, inter, K);
    if (tile == 0) return fail("tc_gated_gemm", "not a shape for the tensor-memory product");
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return fail("tc_gated_gemm", "operands must be 16-byte aligned");
    if (tile == 256) return launch_tc_gated_gemm<256>((const bf16*)x, (const bf16*)w, (bf16*)y, M, inter, K, stream);
    return launch_tc_gated_gemm<192>((const bf16*)x, (const bf16*)w, (bf16*)y, M, inter, K, stream);
}

// Whether the resident-rows kernel takes the product, in the forms that carry half of an RMSNorm.
B200_EXPORT int b200_split_norm_gemm_supports(int M, int N, int K, int gated_inter) {
    const int rows = gated_inter > 0 ? gated_inter : N;
    return (M >= 1 && M <= 16 && K >= 128 && K % 128 == 0 && rows >= 8 && rows % 8 == 0 &&
            b200::slab_smem_bytes(K, gated_inter > 0) <= 200 * 1024) ? 1 : 0;
}

// The resident-rows product with half of an RMSNorm on either side (slab_gemm.cuh), bfloat16 in and out.
//   squares_in != null: x holds rows v * g; the result is multiplied by rsqrt(sum of the row's `pieces`
//   pieces of squares_in[row][...] / K + eps).
//   residual != null (not gated): residual[M][N] += bfloat16(result) in float32, y = residual * weight[N],
//   squares_out[row][N / 8] = sums of the new residual's squares over blocks of eight columns.
B200_EXPORT int b200_split_norm_gemm_bf16(const void* x, const void* w, void* y, int M, int N, int K, int gated_inter,
                                          const void* squares_in, int pieces, float eps, void* residual,
                                          const void* weight, void* squares_out, cudaStream_t stream) {
    using namespace b200;
    if (M == 0 || N == 0) return 0;
    if (!b200_split_norm_gemm_supports(M, N, K, gated_inter)) return fail("split_norm_gemm", "not a shape for the resident-rows kernel");
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y | (uintptr_t)residual | (uintptr_t)weight) & 15)
        return fail("split_norm_gemm", "operands must be 16-byte aligned");
    if (gated_inter > 0 && N != 2 * gated_inter) return fail("split_norm_gemm", "gated product needs N = 2 * inter");
    if (squares_in != nullptr && pieces < 1) return fail("split_norm_gemm", "no pieces of the sums of squares");
    if (residual != nullptr && (gated_inter > 0 || weight == nullptr || squares_out == nullptr))
        return fail("split_norm_gemm", "a residual sum needs the norm's weights and room for the sums of squares, and is not gated");
    SlabNorm norm = {};
    norm.squares_in = static_cast<const float*>(squares_in);
    norm.pieces = pieces;
    norm.eps = eps;
    norm.residual = static_cast<float*>(residual);
    norm.weight = static_cast<const float*>(weight);
    norm.squares_out = static_cast<float*>(squares_out);
    const int rc = launch_slab<bf16>((const bf16*)x, (const bf16*)w, (bf16*)y, M, N, K, gated_inter, stream, norm);
    return rc == 1 ? 0 : (rc < 0 ? rc : fail("split_norm_gemm", "not launched"));
}

// Largest M and the divisibility of K the few-rows kernel takes.
B200_EXPORT int b200_skinny_gemm_supports(int M, int N, int K) {
    return (M >= 1 && M <= 16 && K >= 32 && K % 32 == 0 && N >= 1) ? 1 : 0;
}

// out_dtype: 0 = float32, 1 = bfloat16.  gated_inter > 0: w is [2 * gated_inter, K] and
// y is [M, gated_inter] = silu(x w[:I]^T) * (x w[I:]^T).
B200_EXPORT int b200_skinny_gemm_bf16(const void* x, const void* w, void* y, int M, int N, int K,
                                      int gated_inter, int out_dtype, cudaStream_t stream) {
    using namespace b200;
    if (M == 0 || N == 0) return 0;
    if (!b200_skinny_gemm_supports(M, N, K)) return fail("skinny_gemm", "needs 1 <= M <= 16 and K a multiple of 32");
    if (((uintptr_t)x | (uintptr_t)w) & 15) return fail("skinny_gemm", "operands must be 16-byte aligned");
    if (gated_inter > 0 && N != 2 * gated_inter) return fail("skinny_gemm", "gated product needs N = 2 * inter");
    if ((out_dtype == 0 || out_dtype == 1) && ((uintptr_t)y & (out_dtype == 1 ? 3 : 7)) == 0) {
        const int rc = out_dtype == 1
            ? launch_slab<bf16>((const bf16*)x, (const bf16*)w, (bf16*)y, M, N, K, gated_inter, stream)
            : launch_slab<float>((const bf16*)x, (const bf16*)w, (float*)y, M, N, K, gated_inter, stream);
        if (rc != 0) return rc < 0 ? rc : 0;
    }
    if (out_dtype == 1) {
        if ((uintptr_t)y & 3) return fail("skinny_gemm", "output must be 4-byte aligned");
        return launch_skinny<bf16>((const bf16*)x, (const bf16*)w, (bf16*)y, M, N, K, gated_inter, stream);
    }
    if (out_dtype == 0) {
        if ((uintptr_t)y & 7) return fail("skinny_gemm", "output must be 8-byte aligned");
        return launch_skinny<float>((const bf16*)x, (const bf16*)w, (float*)y, M, N, K, gated_inter, stream);
    }
    return fail("skinny_gemm", "out_dtype must be 0 (float32) or 1 (bfloat16)");
}

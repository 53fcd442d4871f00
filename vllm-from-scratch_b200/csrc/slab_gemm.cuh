// y[M, N] = x[M, K] w[N, K]^T for up to 16 token rows, with a block's whole share of the
// weight matrix resident in shared memory.
//
// A decode step multiplies a handful of token rows by matrices of 8 to 50 MB, one after
// the other, and each such product is short: most of its time is the wait for the first
// bytes.  Weights are written by no kernel, so a block of this kernel asks for all of its
// eight weight rows (K up to 12288: at most 192 KB) with bulk asynchronous copies before
// it waits for the kernel ahead of it on the stream (overlapped launch, common.cuh): the
// matrix is on its way while the short kernel that produces the token rows still runs,
// and everything a block will ever read is in flight at once, with no ring to refill.
// Copies are one per weight row (kSlabQuarters parts of a row, each part with its own
// mbarrier; one part measured best).  Rows have a pitch of K * 2 + 16 bytes, which spreads
// the warps' 16-byte reads over all banks.
// The arithmetic is that of skinny_gemm_kernel (gemm_bf16.cu): m16n8k16 products with the
// token rows as the 16-row operand, the warps splitting K, their sums added in a fixed
// order.  GATED: w is [2 N, K] with N gate rows followed by N up rows; a block holds eight
// of each and stores silu(gate) * up, the feed-forward's first product and activation in one.
// Waits are bounded; a block that gives up sets `error_flag` and stores nothing.
//
// RMSNorm between two such products is split over them, so that no kernel of its own has to read
// and write the rows: rmsnorm(v) g W^T = rsqrt(mean v^2 + eps) * ((v g) W^T) for the norm's
// weights g.  The product ahead of the norm (`SlabNorm::residual` given) adds its rounded result
// into the float32 residual rows v in place (every element has one owner), stores v g instead of
// the result, and the sum of v^2 over its eight columns for every token row to
// squares_out[row][block].  The product behind it (`SlabNorm::squares_in` given) adds these
// pieces up in a fixed order and multiplies its own sums by the root.
#pragma once

#include "async_copy.cuh"

namespace b200 {

constexpr int kSlabWarps = 8;
// Copies per weight row.  One is best: measured 4.9 / 4.0 / 7.7 us for the 4096 x 2048, 2048 x 2048 and
// 2048 x 6144 products against 5.7 / 4.7 / 8.3 us with four and 11.9 / 9.1 / 12.7 us with sixteen: few
// large copies load faster than many small ones, and that outweighs starting on a first part early.
constexpr int kSlabQuarters = 1;
static_assert(128 % (32 * kSlabQuarters) == 0, "the caller checks K % 128 == 0: every part must be whole blocks of 32");
constexpr int kSlabRows = 8;                        // weight rows per block

inline size_t slab_smem_bytes(int K, bool gated) {
    return (size_t)(gated ? 2 : 1) * kSlabRows * ((size_t)K * 2 + 16) + 64 + 128;
}

// WIDE: 9 to 16 token rows (both halves of the 16-row operand are read).
// After the wait a warp's time is round trips to L2 for its fragments of the token rows (the
// weights are in shared memory by then), one per kUnroll blocks of 32 elements of K.
// DEEP: more of them in flight.  Plain form: rows so long (K of 4096 and more) that two blocks
// fill an SM's shared memory, so a block may have the registers of the blocks that do not fit
// (twelve fragments in flight, six for WIDE).  Gated form: eight instead of four.
// The two halves of a split RMSNorm (all null: a plain product).
struct SlabNorm {
    const float* squares_in;        // [rows][pieces]: this product's rows are v g, to be scaled by the root
    int pieces;
    float eps;
    float* residual;                // [M][N] float32, updated in place: this product's result is added to it
    const float* weight;            // [N]: the norm's weights g
    float* squares_out;             // [rows][N / 8]
};

// NORM: which halves of a norm the launch carries (1: squares_in, the root of the norm ahead; 2:
// residual, the sum and the first half of the norm behind; 3: both).  Each is an instantiation of
// its own: the halves cost registers, and these kernels are short enough for that to show.
template <typename OutT, bool GATED, bool WIDE, bool DEEP, int NORM>
__global__ void __launch_bounds__(kSlabWarps * 32, GATED ? 3 : (DEEP ? 2 : 4)) slab_gemm_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, OutT* __restrict__ y, int M, int N,
    int K, int* __restrict__ error_flag, const SlabNorm norm) {
    extern __shared__ __align__(128) unsigned char slab_smem[];
    constexpr int kSets = GATED ? 2 : 1;            // sets of eight rows: gate and up, or one
    __shared__ float partial[kSlabWarps][kSets][32][4];
    __shared__ float row_scale[(NORM & 1) ? 16 : 1];
    overlap_trigger();
    const int pitch = K * 2 + 16;
    unsigned char* rows = slab_smem;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(slab_smem + (((size_t)kSets * kSlabRows * pitch + 63) & ~(size_t)63));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * kSlabRows;
    const int rows_here = min(kSlabRows, N - n0);
    const int quarter_bytes = K * 2 / kSlabQuarters;        // K is a multiple of 128: a multiple of 16 bytes

    if (threadIdx.x == 0) {
        for (int q = 0; q < kSlabQuarters; ++q) mbar_init(bars + q, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // weight rows past the end of the matrix read as zeros
    for (int set = 0; set < kSets; ++set)
        for (int i = threadIdx.x; i < (kSlabRows - rows_here) * (pitch / 16); i += blockDim.x)
            reinterpret_cast<uint4*>(rows + (size_t)(set * kSlabRows + rows_here) * pitch)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    if (warp == 0) {
        if (lane == 0)
            for (int q = 0; q < kSlabQuarters; ++q) mbar_expect_tx(bars + q, (unsigned)(kSets * rows_here * quarter_bytes));
        __syncwarp();
        const int set = lane / kSlabRows, r = lane % kSlabRows;       // lanes 8..15: the up rows, N rows further on
        if (set < kSets && r < rows_here) {
            const unsigned char* src = reinterpret_cast<const unsigned char*>(w + ((size_t)set * N + n0 + r) * K);
            for (int q = 0; q < kSlabQuarters; ++q)
                bulk_copy_g2s(rows + (size_t)lane * pitch + q * quarter_bytes, src + q * quarter_bytes,
                              (unsigned)quarter_bytes, bars + q);
        }
    }
    overlap_wait();                                 // the token rows come from the kernel before this one

    constexpr bool kScaled = (NORM & 1) != 0, kFolded = (NORM & 2) != 0;

    // What the warp that stores will add to, asked for ahead of the products.
    float2 before[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)}, gain = make_float2(0.0f, 0.0f);
    if (kFolded && warp == 0) {
#pragma unroll
        for (int half = 0; half < (WIDE ? 2 : 1); ++half)
            if (g + half * 8 < M)
                before[half] = __ldcg(reinterpret_cast<const float2*>(norm.residual + (size_t)(g + half * 8) * N + n0 + 2 * t));
        gain = *reinterpret_cast<const float2*>(norm.weight + n0 + 2 * t);
    }

    const bool x_ok = g < M, x_hi_ok = WIDE && g + 8 < M;   // rows g and g + 8 of the 16-row operand
    const __nv_bfloat16* x_row = x + (size_t)(x_ok ? g : 0) * K + 8 * t;
    const __nv_bfloat16* x_row_hi = x + (size_t)(x_hi_ok ? g + 8 : 0) * K + 8 * t;
    const unsigned char* w_row = rows + (size_t)g * pitch + 16 * t;
    float acc[kSets][4];
#pragma unroll
    for (int set = 0; set < kSets; ++set) acc[set][0] = acc[set][1] = acc[set][2] = acc[set][3] = 0.0f;
    const int blocks = K >> 5;                      // blocks of 32 elements of K
    const int blocks_per_quarter = blocks / kSlabQuarters;        // K a multiple of 128 (checked by the caller)
    const uint4 zero = make_uint4(0, 0, 0, 0);
    bool ok = true;
    constexpr int kUnroll = GATED ? (WIDE ? 2 : (DEEP ? 8 : 4)) : (DEEP ? (WIDE ? 6 : 12) : (WIDE ? 2 : 4));
    for (int q = 0; q < kSlabQuarters; ++q) {
        const int first = q * blocks_per_quarter, last = first + blocks_per_quarter;
        bool waited = false;
        for (int j = first + warp; j < last; j += kUnroll * kSlabWarps) {
            uint4 xv[kUnroll], xh[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int block = j + u * kSlabWarps;
                xv[u] = (block < last && x_ok) ? *reinterpret_cast<const uint4*>(x_row + (block << 5)) : zero;
                xh[u] = (WIDE && block < last && x_hi_ok) ? *reinterpret_cast<const uint4*>(x_row_hi + (block << 5)) : zero;
            }
            if (!waited) {
                if (ok && !mbar_wait(bars + q, 0)) { atomicExch(error_flag, 41); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
                waited = true;
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int block = j + u * kSlabWarps;
                if (block >= last) break;
#pragma unroll
                for (int set = 0; set < kSets; ++set) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(w_row + (size_t)set * kSlabRows * pitch + (size_t)block * 64);
                    mma_bf16_16816(acc[set], xv[u].x, xh[u].x, xv[u].y, xh[u].y, wv.x, wv.y);
                    mma_bf16_16816(acc[set], xv[u].z, xh[u].z, xv[u].w, xh[u].w, wv.z, wv.w);
                }
            }
        }
    }
    // Every copy must have landed before the block may leave (its shared memory is theirs).
    for (int q = 0; q < kSlabQuarters; ++q)
        if (ok && !mbar_wait(bars + q, 0)) { atomicExch(error_flag, 42); ok = false; }
    ok = __all_sync(0xffffffffu, ok);

#pragma unroll
    for (int set = 0; set < kSets; ++set)
#pragma unroll
        for (int e = 0; e < 4; ++e) partial[warp][set][lane][e] = acc[set][e];
    // The root of the norm ahead: warp r adds the pieces of token row r's sum of squares, a lane
    // every 32nd piece, then the lanes' sums in the order of the shuffles.  (Asked for here, after
    // the products: held in registers across them, the pieces cost more than their round trip.)
    for (int row = warp; kScaled && row < 16; row += kSlabWarps) {
        float scale = 1.0f;
        if (row < M) {
            const float* mine = norm.squares_in + (size_t)row * norm.pieces;
            float sum = 0.0f;
            for (int i = lane; i < norm.pieces; i += 32) sum += __ldcg(mine + i);
            scale = rsqrtf(warp_sum(sum) / (float)K + norm.eps);
        }
        if (lane == 0) row_scale[row] = scale;
    }
    __syncthreads();
    if (warp != 0 || !ok) return;
    // accumulator layout: c0, c1 = (token g, weight rows 2t, 2t + 1), c2, c3 = (token g + 8, same rows)
    constexpr int kHalves = WIDE ? 2 : 1;
    const int n = n0 + 2 * t;
#pragma unroll
    for (int half = 0; half < kHalves; ++half) {
        float total[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float sums[kSets];
#pragma unroll
            for (int set = 0; set < kSets; ++set) {
                float sum = partial[0][set][lane][half * 2 + e];
#pragma unroll
                for (int wi = 1; wi < kSlabWarps; ++wi) sum += partial[wi][set][lane][half * 2 + e];
                sums[set] = sum;
            }
            const float scale = kScaled ? row_scale[g + half * 8] : 1.0f;
            const float first = sums[0] * scale;
            total[e] = GATED ? first / (1.0f + expf(-first)) * (sums[kSets - 1] * scale) : first;
        }
        const int token = g + half * 8;
        if (kFolded) {
            // (the launcher gives this form whole blocks of eight columns and an even N)
            float squares = 0.0f;
            if (token < M) {
                const float2 v = make_float2(before[half].x + to_float(from_float<OutT>(total[0])),
                                             before[half].y + to_float(from_float<OutT>(total[1])));
                *reinterpret_cast<float2*>(norm.residual + (size_t)token * N + n) = v;
                total[0] = v.x * gain.x;
                total[1] = v.y * gain.y;
                squares = v.x * v.x + v.y * v.y;
            }
            squares += __shfl_xor_sync(0xffffffffu, squares, 1);
            squares += __shfl_xor_sync(0xffffffffu, squares, 2);
            if (t == 0 && token < M) norm.squares_out[(size_t)token * gridDim.x + blockIdx.x] = squares;
        }
        if (token >= M) continue;
        OutT* dst = y + (size_t)token * N + n;
        if (n + 1 < N && (N & 1) == 0) store_pair<OutT>(dst, total[0], total[1]);
        else {
            if (n < N) store_one<OutT>(dst, total[0]);
            if (n + 1 < N) store_one<OutT>(dst + 1, total[1]);
        }
    }
}

}  // namespace b200

// Few-rows bfloat16 product as a stream of bulk copies: y[M, N] = x[M, K] . w[N, K]^T,
// M <= 16, float32 accumulation.
//
// Persistent blocks.  A producer thread walks the block's share of the weight
// matrix (tiles of 8 rows, or 8 gate + 8 up rows, by chunks of 512 columns) and
// brings every row segment (1 KB, contiguous in memory) into a ring of shared
// memory stages with one bulk asynchronous copy (cp.async.bulk), each stage
// guarded by a "full" mbarrier that counts the bytes landed.  Four consumer warps
// take the stages in order, each a quarter of the chunk's k-blocks, multiply on the
// tensor cores against the token rows (read through L1, where they stay for all of
// a block's tiles) and hand the stage back through an "empty" mbarrier.  The copy
// engine thereby keeps many kilobytes per SM in flight with a handful of
// instructions.
//
// Measured on B200 (M = 8, bfloat16): with 1 KB copies this kernel reaches about
// 2.5 TB/s on a 50 MB matrix, bound by the rate at which one thread can issue bulk
// copies, where the plain-load kernel in gemm_bf16.cu reaches 3.2 TB/s; it wins only
// on small matrices (2048 x 2048: 5.1 us against 6.1 us).  It is therefore not the
// default: gemm_bf16.cu uses it only when the environment variable
// B200_STREAM_GEMM is set.  A version that moves 8 x 512 tiles with one tensor copy
// each (cp.async.bulk.tensor) would need an order of magnitude fewer copies.
//
// Rows of a stage are 1088 bytes apart (1024 + 64), which spreads the eight rows a
// warp reads together over all shared-memory banks.
//
// Every wait on an mbarrier is bounded: after kWaitLimit failed polls the waiter
// records a code in `error_flag` and leaves; the producer then still waits (bounded)
// for the copies it started before the block exits.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kStreamChunk = 512;                       // columns per row per stage
constexpr int kStreamPitch = kStreamChunk * 2 + 64;     // bytes between rows of a stage
constexpr int kStreamConsumers = 4;                     // warps
constexpr int kStreamBlocksPerWarp = kStreamChunk / 32 / kStreamConsumers;
constexpr int kWaitLimit = 1 << 20;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait; false after kWaitLimit polls.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity) {
    for (int i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, unsigned bytes, void* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                               unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void stream_store(T* p, float a, float b, bool two);
template <> __device__ __forceinline__ void stream_store<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, bool two) {
    if (two && ((uintptr_t)p & 3) == 0) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
    else { p[0] = __float2bfloat16_rn(a); if (two) p[1] = __float2bfloat16_rn(b); }
}
template <> __device__ __forceinline__ void stream_store<float>(float* p, float a, float b, bool two) {
    p[0] = a;
    if (two) p[1] = b;
}

// TILES = 1: a tile is 8 weight rows.  TILES = 2 with GATED: 8 gate rows and the 8 up
// rows `up_offset` below them; without GATED: 16 consecutive rows.
// The token rows are copied into shared memory once per block (x_rows = 8 or 16 rows
// of 2 K + 64 bytes), then the ring of STAGES weight stages follows.
template <int TILES, bool GATED, typename OutT>
__global__ void __launch_bounds__((kStreamConsumers + 1) * 32) stream_gemm_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, OutT* __restrict__ y,
    int M, int N, int K, int up_offset, int num_tiles, int STAGES, int x_rows,
    int* __restrict__ error_flag) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int kRows = 8 * TILES;
    constexpr int kStageBytes = kRows * kStreamPitch;
    const int x_pitch = 2 * K + 64;
    unsigned char* x_s = smem;
    unsigned char* stages = smem + (size_t)x_rows * x_pitch;
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(stages + (size_t)STAGES * kStageBytes);
    unsigned long long* empty_bar = full_bar + STAGES;
    unsigned long long* x_bar = empty_bar + STAGES;
    float* partial = reinterpret_cast<float*>(x_bar + 1);               // [2][consumers][TILES][32][4]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kStreamConsumers);
        }
        mbar_init(x_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const int chunks = (K + kStreamChunk - 1) / kStreamChunk;
    const int rows_per_tile = GATED ? 8 : kRows;                // output columns a tile covers

    if (warp == kStreamConsumers) {
        // ------------------------------------------------------------- producer
        if (lane != 0) return;
        mbar_expect_tx(x_bar, (unsigned)M * (unsigned)K * 2u);
        for (int r = 0; r < M; ++r) bulk_copy_g2s(x_s + (size_t)r * x_pitch, x + (size_t)r * K, (unsigned)K * 2u, x_bar);
        int step = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int n0 = tile * rows_per_tile;
            for (int c = 0; c < chunks && ok; ++c, ++step) {
                const int s = step % STAGES;
                const unsigned phase = (step / STAGES) & 1;
                if (step >= STAGES && !mbar_wait(empty_bar + s, phase ^ 1)) {
                    atomicExch(error_flag, 1);
                    ok = false;
                    break;
                }
                const int k0 = c * kStreamChunk;
                const unsigned bytes = (unsigned)min(kStreamChunk, K - k0) * 2u;
                int valid = 0;
                for (int r = 0; r < kRows; ++r) {
                    const int n = GATED ? n0 + (r & 7) : n0 + r;
                    if (n < N) ++valid;
                }
                mbar_expect_tx(full_bar + s, bytes * valid);
                unsigned char* dst = stages + (size_t)s * kStageBytes;
                for (int r = 0; r < kRows; ++r) {
                    const int n = GATED ? n0 + (r & 7) : n0 + r;
                    if (n >= N) continue;
                    const size_t row = GATED ? (size_t)n + (size_t)(r >> 3) * up_offset : (size_t)n;
                    bulk_copy_g2s(dst + r * kStreamPitch, w + row * K + k0, bytes, full_bar + s);
                }
            }
        }
        // Copies this thread started must have landed before the block's shared memory goes away.
        const int first = step > STAGES ? step - STAGES : 0;
        for (int done = first; done < step; ++done)
            if (!mbar_wait(full_bar + done % STAGES, (done / STAGES) & 1)) atomicExch(error_flag, 2);
        if (!mbar_wait(x_bar, 0)) atomicExch(error_flag, 2);
        return;
    }

    // ----------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const bool x_lo = g < M, x_hi = g + 8 < M;
    const unsigned char* x_row_lo = x_s + (size_t)(x_lo ? g : 0) * x_pitch + 16 * t;
    const unsigned char* x_row_hi = x_s + (size_t)(x_hi ? g + 8 : 0) * x_pitch + 16 * t;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    int step = 0;
    int tile_count = 0;
    bool ok = true;
    if (!mbar_wait(x_bar, 0)) {
        atomicExch(error_flag, 3);
        ok = false;
    }
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tile_count) {
        float acc[TILES][4];
#pragma unroll
        for (int i = 0; i < TILES; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
        for (int c = 0; c < chunks; ++c, ++step) {
            const int s = step % STAGES;
            const unsigned phase = (step / STAGES) & 1;
            const int k0 = c * kStreamChunk;
            const int blocks = min(kStreamChunk, K - k0) >> 5;
            if (ok && !mbar_wait(full_bar + s, phase)) {
                atomicExch(error_flag, 3);
                ok = false;            // no more waiting or arithmetic, but keep every rendezvous
            }
            const unsigned char* base = stages + (size_t)s * kStageBytes + g * kStreamPitch + t * 16;
#pragma unroll 4
            for (int u = 0; u < kStreamBlocksPerWarp; ++u) {
                const int j = warp + u * kStreamConsumers;
                if (j < blocks && ok) {
                    const uint4 xl = x_lo ? *reinterpret_cast<const uint4*>(x_row_lo + 2 * k0 + (j << 6)) : zero;
                    const uint4 xh = x_hi ? *reinterpret_cast<const uint4*>(x_row_hi + 2 * k0 + (j << 6)) : zero;
#pragma unroll
                    for (int i = 0; i < TILES; ++i) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(base + i * 8 * kStreamPitch + (j << 6));
                        mma_bf16_16816(acc[i], xl.x, xh.x, xl.y, xh.y, wv.x, wv.y);
                        mma_bf16_16816(acc[i], xl.z, xh.z, xl.w, xh.w, wv.z, wv.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + s);
        }
        // the four warps' sums of this tile, added in a fixed order by warp 0
        float* mine = partial + ((size_t)(tile_count & 1) * kStreamConsumers + warp) * TILES * 128;
#pragma unroll
        for (int i = 0; i < TILES; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[(i * 32 + lane) * 4 + e] = acc[i][e];
        asm volatile("bar.sync 1, %0;\n" ::"n"(kStreamConsumers * 32) : "memory");
        if (warp != 0 || !ok) continue;
        const float* all = partial + (size_t)(tile_count & 1) * kStreamConsumers * TILES * 128;
        float total[TILES][4];
#pragma unroll
        for (int i = 0; i < TILES; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float sum = all[(i * 32 + lane) * 4 + e];
#pragma unroll
                for (int wi = 1; wi < kStreamConsumers; ++wi) sum += all[((size_t)wi * TILES * 32 + i * 32 + lane) * 4 + e];
                total[i][e] = sum;
            }
        // c0, c1 = (token g, weight rows 2t, 2t+1 of the 8-row block); c2, c3 = (token g + 8, same rows)
        const int n0 = tile * rows_per_tile;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int token = g + half * 8;
            if (token >= M) continue;
            if (GATED) {
                const int n = n0 + 2 * t;
                if (n >= N) continue;
                const float g0 = total[0][half * 2], g1 = total[0][half * 2 + 1];
                const float u0 = total[TILES - 1][half * 2], u1 = total[TILES - 1][half * 2 + 1];
                stream_store<OutT>(y + (size_t)token * N + n, g0 / (1.0f + expf(-g0)) * u0,
                                   g1 / (1.0f + expf(-g1)) * u1, n + 1 < N);
            } else {
#pragma unroll
                for (int i = 0; i < TILES; ++i) {
                    const int n = n0 + i * 8 + 2 * t;
                    if (n >= N) continue;
                    stream_store<OutT>(y + (size_t)token * N + n, total[i][half * 2], total[i][half * 2 + 1], n + 1 < N);
                }
            }
        }
    }
}

// Shared memory of one block: token rows, weight stages, barriers, partial sums.
inline int stream_gemm_smem(int tiles, int stages, int x_rows, int K) {
    return x_rows * (2 * K + 64) + stages * 8 * tiles * kStreamPitch + (2 * stages + 1) * 8 +
           2 * kStreamConsumers * tiles * 128 * 4;
}

}  // namespace b200

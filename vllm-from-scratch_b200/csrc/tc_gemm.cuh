// bfloat16 product on the 5th-generation tensor cores for up to 256 token rows:
// y[M, N] = x[M, K] . w[N, K]^T, float32 accumulation in tensor memory.
//
// The product is computed transposed ("swap A/B"): a block owns 128 rows of the
// weight matrix, which become the M = 128 rows of a tcgen05.mma, and all token
// rows (padded to a multiple of 16) are its N columns.  With few tokens the kernel
// is a stream of the weight matrix, so its shape follows the copy engine:
//   * one producer thread issues tensor copies (TMA): a 128 x 64 tile of w (16 KB,
//     128-byte swizzle) and the matching tile of x per k-step into a ring of stages;
//   * one thread issues the MMAs (four K = 16 steps per stage) straight from shared
//     memory descriptors; tcgen05.commit hands a stage back when they have read it;
//   * K may be split over several blocks (grid.y) so that small matrices still fill
//     the GPU; each split writes its float32 partial block, the last block to arrive
//     for a row tile adds the partials in a fixed order (the result does not depend
//     on arrival order) and writes the output;
//   * the accumulator is read back with tcgen05.ld, 32 lanes per warp.
// The gated variant loads 64 gate rows and the 64 up rows that go with them into
// one tile and writes silu(gate) * up.
//
// All mbarrier waits are bounded (see stream_gemm.cuh); on a timeout the block
// records a code, skips its arithmetic, still frees its tensor memory and leaves.
#pragma once

#include <cuda.h>

#include "stream_gemm.cuh"

namespace b200 {

constexpr int kTcRows = 128;          // weight rows per block = UMMA M
constexpr int kTcK = 64;              // k elements per stage (one 128-byte swizzle row)
constexpr int kTcATile = kTcRows * kTcK * 2;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile, int byte_offset) {
    const unsigned address = (smem_u32(smem_tile) + byte_offset) & 0x3FFFF;
    unsigned long long desc = 0;
    desc |= (unsigned long long)(address >> 4);                 // start address, 16-byte units
    desc |= (unsigned long long)1 << 16;                        // leading byte offset (unused with swizzle)
    desc |= (unsigned long long)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    desc |= (unsigned long long)1 << 46;                        // descriptor version of this architecture
    desc |= (unsigned long long)2 << 61;                        // 128-byte swizzle
    return desc;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(kTcRows >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a, unsigned long long b,
                                          unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory layout (offsets from a 1024-byte aligned base).
struct TcLayout {
    int stages, ntok, b_tile;
    __host__ __device__ TcLayout(int stages_, int ntok_) : stages(stages_), ntok(ntok_), b_tile(ntok_ * kTcK * 2) {}
    __host__ __device__ int a(int s) const { return s * (kTcATile + b_tile); }
    __host__ __device__ int b(int s) const { return a(s) + kTcATile; }
    __host__ __device__ int barriers() const { return stages * (kTcATile + b_tile); }
    __host__ __device__ int exchange() const { return barriers() + (2 * stages + 1) * 8 + 16; }   // gated: [64][ntok] floats
    __host__ __device__ int total(bool gated) const { return exchange() + (gated ? 64 * ntok * 4 : 0) + 1024; }
};

// grid (row tiles, splits).  `scratch` holds splits x M x N floats when splits > 1,
// `counters` one int per row tile (zero between launches).
template <bool GATED, typename OutT>
__global__ void __launch_bounds__(128) tc_gemm_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    float* __restrict__ scratch, int* __restrict__ counters, OutT* __restrict__ y, int M, int N, int K,
    int ntok, int stages, int steps_per_split, int up_offset, int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const TcLayout layout(stages, ntok);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + layout.barriers());
    unsigned long long* empty_bar = full_bar + stages;
    unsigned long long* done_bar = empty_bar + stages;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(done_bar + 1);
    int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);
    float* exchange = reinterpret_cast<float*>(smem + layout.exchange());

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int total_steps = (K + kTcK - 1) / kTcK;
    const int step_begin = split * steps_per_split;
    const int step_end = min(total_steps, step_begin + steps_per_split);
    const int my_steps = max(0, step_end - step_begin);
    const int rows_per_tile = GATED ? 64 : kTcRows;          // output columns a tile covers
    const int row0 = tile * rows_per_tile;
    int tmem_cols = 32;
    while (tmem_cols < ntok) tmem_cols *= 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"(tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_d = *tmem_slot;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ producer
        const unsigned stage_bytes = kTcATile + layout.b_tile;
        for (int i = 0; i < my_steps; ++i) {
            const int s = i % stages;
            if (i >= stages && !mbar_wait(empty_bar + s, ((i / stages) & 1) ^ 1)) {
                atomicExch(error_flag, 11);
                ok = false;
                break;
            }
            const int k0 = (step_begin + i) * kTcK;
            mbar_expect_tx(full_bar + s, stage_bytes);
            if (GATED) {
                tma_load_2d(smem + layout.a(s), &map_w, k0, row0, full_bar + s);
                tma_load_2d(smem + layout.a(s) + kTcATile / 2, &map_w, k0, up_offset + row0, full_bar + s);
            } else {
                tma_load_2d(smem + layout.a(s), &map_w, k0, row0, full_bar + s);
            }
            tma_load_2d(smem + layout.b(s), &map_x, k0, 0, full_bar + s);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        const unsigned idesc = umma_idesc(ntok);
        for (int i = 0; i < my_steps; ++i) {
            const int s = i % stages;
            if (!mbar_wait(full_bar + s, (i / stages) & 1)) {
                atomicExch(error_flag, 12);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int j = 0; j < kTcK / 16; ++j)
                umma_bf16(tmem_d, umma_desc(smem + layout.a(s), j * 32), umma_desc(smem + layout.b(s), j * 32),
                          idesc, i > 0 || j > 0);
            umma_commit(empty_bar + s);          // the stage is free once these MMAs have read it
        }
        umma_commit(done_bar);                   // arrives when every MMA above has finished
    }
    __syncwarp();

    // ------------------------------------------------------------------ epilogue
    if (my_steps > 0 && !mbar_wait(done_bar, 0)) {
        atomicExch(error_flag, 13);
        ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);        // tcgen05.ld below is a whole-warp instruction
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int row = warp * 32 + lane;                        // row of the tile = lane of tensor memory
    const int chunks = ntok / 16;
    const bool gate_half = row < 64;
    // Which output column (weight row) this thread's accumulator row stands for.
    const int n = GATED ? row0 + (row & 63) : row0 + row;
    const bool n_ok = n < N;

    if (splits > 1) {
        // partial sums of this split: scratch[split][token][n]; the gated tile keeps gate and up apart
        float* mine = scratch + (size_t)split * M * (GATED ? 2 * N : N);
        for (int c = 0; c < chunks; ++c) {
            float v[16];
            if (my_steps > 0 && ok) tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + c * 16, v);
            else
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int token = c * 16 + e;
                if (token < M && n_ok)
                    mine[(size_t)token * (GATED ? 2 * N : N) + (GATED && !gate_half ? N : 0) + n] = v[e];
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int before = atomicAdd(counters + tile, 1);
            *last_flag = before == splits - 1;
            if (before == splits - 1) counters[tile] = 0;    // ready for the next launch
        }
        __syncthreads();
        if (*last_flag) {
            __threadfence();
            const int width = GATED ? 2 * N : N;
            // 128 threads walk the tile's outputs: thread = output column, loop over tokens
            for (int idx = threadIdx.x; idx < rows_per_tile * M; idx += blockDim.x) {
                const int token = idx / rows_per_tile, col = row0 + idx % rows_per_tile;
                if (col >= N) continue;
                float sum = 0.0f, sum_up = 0.0f;
                for (int s = 0; s < splits; ++s) {
                    const float* part = scratch + ((size_t)s * M + token) * width;
                    sum += part[col];
                    if (GATED) sum_up += part[N + col];
                }
                const float result = GATED ? sum / (1.0f + expf(-sum)) * sum_up : sum;
                y[(size_t)token * N + col] = from_float<OutT>(result);
            }
        }
    } else {
        for (int c = 0; c < chunks; ++c) {
            float v[16];
            if (ok) tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + c * 16, v);
            else
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.0f;
            if (GATED) {
                // rows 64..127 hold the up values of the columns whose gate values sit in rows 0..63
                if (!gate_half)
#pragma unroll
                    for (int e = 0; e < 16; ++e) exchange[(row - 64) * 16 + e] = v[e];
                __syncthreads();
                if (gate_half && n_ok)
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int token = c * 16 + e;
                        if (token < M) {
                            const float up = exchange[row * 16 + e];
                            y[(size_t)token * N + n] = from_float<OutT>(v[e] / (1.0f + expf(-v[e])) * up);
                        }
                    }
                __syncthreads();
            } else if (n_ok) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const int token = c * 16 + e;
                    if (token < M) y[(size_t)token * N + n] = from_float<OutT>(v[e]);
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(tmem_cols));
}

}  // namespace b200

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
//   * K may be split over the blocks of a thread-block cluster (grid.y = cluster size,
//     at most 8) so that small matrices still fill the GPU: every block leaves its
//     float32 partial tile in its own shared memory, and after a cluster barrier each
//     block adds, for its share of the tokens, the partial tiles of all blocks through
//     distributed shared memory, in the order of the splits (the result does not depend
//     on which block finished first), and writes those rows of the output;
//   * the accumulator is read back with tcgen05.ld, 32 lanes per warp;
//   * launched overlapped (common.cuh): the weight tiles of the first stages, which no
//     kernel writes, are requested before the wait on the kernel ahead on the stream.
// The gated variant loads 64 gate rows and the 64 up rows that go with them into
// one tile and writes silu(gate) * up.
//
// All mbarrier waits are bounded (see stream_gemm.cuh); on a timeout the block
// records a code, skips its arithmetic, still frees its tensor memory and leaves.
#pragma once

#include "tcgen05.cuh"

namespace b200 {

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned cluster_size() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
    return r;
}
// Every thread of every block of the cluster arrives and waits; writes to shared memory
// before it are visible to the cluster's other blocks after it.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Address, in the cluster's shared window, of `local` (an address in this block's shared
// memory) in the block of rank `rank`.
__device__ __forceinline__ unsigned cluster_address(unsigned local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ float cluster_load(unsigned address) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(address) : "memory");
    return v;
}

__device__ __forceinline__ float4 cluster_load4(unsigned address) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(address)
                 : "memory");
    return v;
}

constexpr int kTcMaxSplits = 8;       // the portable cluster size
constexpr int kTcHeader = 1024;       // barriers and the tensor-memory slot, ahead of the tiles

// Shared-memory layout (offsets from a 1024-byte aligned base): header, then the ring of
// stages; the float32 partial tile [ntok][128] of the split-K sum lies over the ring,
// which nothing reads any more by then.
struct TcLayout {
    int stages, ntok, b_tile;
    __host__ __device__ TcLayout(int stages_, int ntok_) : stages(stages_), ntok(ntok_), b_tile(ntok_ * kTcK * 2) {}
    __host__ __device__ int stage_bytes() const { return kTcATile + b_tile; }
    __host__ __device__ int a(int s) const { return kTcHeader + s * stage_bytes(); }
    __host__ __device__ int b(int s) const { return a(s) + kTcATile; }
    __host__ __device__ int partial() const { return kTcHeader; }
    __host__ __device__ int total() const {
        const int ring = stages * stage_bytes(), tile = ntok * kTcRows * 4;
        return kTcHeader + (ring > tile ? ring : tile) + 1024;       // 1024: room to align the base
    }
};

// Sum over the RANKS partial tiles of a cluster for this block's share of the tokens, and store.
// Tokens go in fours: four warps, one token each, a lane takes four floats of its line (gated:
// gate and up of two columns).  The block of rank r sums the fours r, r + RANKS, ...; the loads
// of about sixteen (four, split) pairs are in flight together, since each crosses the cluster.
template <bool GATED, typename OutT, int RANKS>
__device__ __forceinline__ void tc_sum_splits(const float* partial, OutT* __restrict__ y, int M, int N, int row0,
                                              int rank) {
    constexpr int kBatch = 16 / RANKS;
    constexpr int kOut = GATED ? 2 : 4;                      // outputs per thread and token
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = row0 + lane * kOut;
    unsigned remote[RANKS];
#pragma unroll
    for (int s = 0; s < RANKS; ++s) remote[s] = cluster_address(smem_u32(partial), (unsigned)s) + lane * 16;
    const bool vector_store = (N % kOut) == 0;               // every row of y then starts on a multiple of kOut
    for (int four0 = rank; four0 * 4 < M; four0 += kBatch * RANKS) {
        float4 part[kBatch][RANKS];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int token = (four0 + b * RANKS) * 4 + warp;
#pragma unroll
            for (int s = 0; s < RANKS; ++s)
                part[b][s] = token < M ? cluster_load4(remote[s] + token * (kTcRows * 4))
                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int token = (four0 + b * RANKS) * 4 + warp;
            float4 sum = part[b][0];
#pragma unroll
            for (int s = 1; s < RANKS; ++s) {
                sum.x += part[b][s].x;
                sum.y += part[b][s].y;
                sum.z += part[b][s].z;
                sum.w += part[b][s].w;
            }
            if (token >= M || n >= N) continue;
            float result[4] = {sum.x, sum.y, sum.z, sum.w};
            if (GATED) {
                result[0] = sum.x / (1.0f + expf(-sum.x)) * sum.y;
                result[1] = sum.z / (1.0f + expf(-sum.z)) * sum.w;
            }
            OutT* dst = y + (size_t)token * N + n;
            if (vector_store) {          // n + kOut <= N follows from n < N
                store_pair<OutT>(dst, result[0], result[1]);
                if (!GATED) store_pair<OutT>(dst + 2, result[2], result[3]);
            } else {
#pragma unroll
                for (int e = 0; e < kOut; ++e)
                    if (n + e < N) dst[e] = from_float<OutT>(result[e]);
            }
        }
    }
}

// grid (row tiles, splits), cluster (1, splits, 1): the blocks of a cluster share a row
// tile and take consecutive ranges of `steps_per_split` k-steps.
template <bool GATED, typename OutT>
__global__ void __launch_bounds__(128) tc_gemm_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, OutT* __restrict__ y,
    int M, int N, int K, int ntok, int stages, int steps_per_split, int up_offset, int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    // The same offset in every block of the cluster: the dynamic shared memory of all of them starts at the
    // same address of the shared window, so what is rounded up here is rounded alike everywhere.
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const TcLayout layout(stages, ntok);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem);
    unsigned long long* empty_bar = full_bar + stages;
    unsigned long long* done_bar = empty_bar + stages;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(done_bar + 1);
    float* partial = reinterpret_cast<float*>(smem + layout.partial());

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank(), ranks = (int)cluster_size();
    const int tile = blockIdx.x;
    const int total_steps = (K + kTcK - 1) / kTcK;
    const int step_begin = rank * steps_per_split;
    const int step_end = min(total_steps, step_begin + steps_per_split);
    const int my_steps = max(0, step_end - step_begin);
    constexpr int kColumns = GATED ? 64 : kTcRows;           // output columns a tile covers
    const int row0 = tile * kColumns;
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
    // Only now may blocks of the next kernel be scheduled beside this one: one that took tensor memory
    // first and then waited for this kernel to end would leave this block waiting for columns for ever.
    // (Blocks of this kernel cannot fill an SM's tensor memory among themselves: see tc_plan.)
    overlap_trigger();

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------ producer
        auto load_w = [&](int i, int s) {
            const int k0 = (step_begin + i) * kTcK;
            if (GATED) {
                tma_load_2d(smem + layout.a(s), &map_w, k0, row0, full_bar + s);
                tma_load_2d(smem + layout.a(s) + kTcATile / 2, &map_w, k0, up_offset + row0, full_bar + s);
            } else {
                tma_load_2d(smem + layout.a(s), &map_w, k0, row0, full_bar + s);
            }
        };
        // Weights are written by no kernel: the first stages' tiles are on their way
        // while the kernel that produces the token rows still runs.
        const int early = min(my_steps, stages);
        for (int i = 0; i < early; ++i) {
            mbar_expect_tx(full_bar + i, (unsigned)layout.stage_bytes());
            load_w(i, i);
        }
        overlap_wait();
        for (int i = 0; i < early; ++i)
            tma_load_2d(smem + layout.b(i), &map_x, (step_begin + i) * kTcK, 0, full_bar + i);
        for (int i = early; i < my_steps; ++i) {
            const int s = i % stages;
            if (!mbar_wait(empty_bar + s, ((i / stages) & 1) ^ 1)) {
                atomicExch(error_flag, 11);
                ok = false;
                break;
            }
            mbar_expect_tx(full_bar + s, (unsigned)layout.stage_bytes());
            load_w(i, s);
            tma_load_2d(smem + layout.b(s), &map_x, (step_begin + i) * kTcK, 0, full_bar + s);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        const unsigned idesc = umma_idesc(ntok);
        const unsigned long long desc_a = umma_desc(smem + layout.a(0), 0), desc_b = umma_desc(smem + layout.b(0), 0);
        const unsigned stage_units = (unsigned)layout.stage_bytes() >> 4;     // descriptors count 16-byte units
        for (int i = 0; i < my_steps; ++i) {
            const int s = i % stages;
            if (!mbar_wait(full_bar + s, (i / stages) & 1)) {
                atomicExch(error_flag, 12);
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned long long a = desc_a + s * stage_units, b = desc_b + s * stage_units;
#pragma unroll
            for (int j = 0; j < kTcK / 16; ++j)      // 16 elements of K further on: 32 bytes, two units
                umma_bf16(tmem_d, a + 2 * j, b + 2 * j, idesc, i > 0 || j > 0);
            umma_commit(empty_bar + s);          // the stage is free once these MMAs have read it
        }
        umma_commit(done_bar);                   // arrives when every MMA above has finished
    }
    __syncwarp();

    // ------------------------------------------------ partial tile to shared memory
    if (my_steps > 0 && !mbar_wait(done_bar, 0)) {
        atomicExch(error_flag, 13);
        ok = false;
    }
    ok = __all_sync(0xffffffffu, ok);        // tcgen05.ld below is a whole-warp instruction
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    overlap_wait();                          // nothing is stored before the kernel ahead has ended
    const int row = warp * 32 + lane;        // row of the tile = lane of tensor memory
    if (!GATED && ranks == 1) {
        // One block has the whole sum: from tensor memory straight to the output.
        const int n = row0 + row;
        for (int c = 0; c * 16 < M; ++c) {
            float v[16];
            if (ok) tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + c * 16, v);
            else
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.0f;
            if (n < N)
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (c * 16 + e < M) y[(size_t)(c * 16 + e) * N + n] = from_float<OutT>(v[e]);
        }
    } else {
        // A token's 128 sums form one line of the partial tile; the gated tile's lines hold
        // gate and up of a column side by side (rows r and 64 + r of the accumulator).
        const int place = GATED ? (((row & 63) << 1) | (row >> 6)) : row;
        for (int c = 0; c * 16 < M; ++c) {
            float v[16];
            if (my_steps > 0 && ok) tmem_ld16(tmem_d + ((unsigned)(warp * 32) << 16) + c * 16, v);
            else
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) partial[(c * 16 + e) * kTcRows + place] = v[e];
        }
        if (ranks > 1) cluster_barrier();
        else __syncthreads();
        switch (ranks) {
            case 1: tc_sum_splits<GATED, OutT, 1>(partial, y, M, N, row0, rank); break;
            case 2: tc_sum_splits<GATED, OutT, 2>(partial, y, M, N, row0, rank); break;
            case 3: tc_sum_splits<GATED, OutT, 3>(partial, y, M, N, row0, rank); break;
            case 4: tc_sum_splits<GATED, OutT, 4>(partial, y, M, N, row0, rank); break;
            case 5: tc_sum_splits<GATED, OutT, 5>(partial, y, M, N, row0, rank); break;
            case 6: tc_sum_splits<GATED, OutT, 6>(partial, y, M, N, row0, rank); break;
            case 7: tc_sum_splits<GATED, OutT, 7>(partial, y, M, N, row0, rank); break;
            default: tc_sum_splits<GATED, OutT, 8>(partial, y, M, N, row0, rank); break;
        }
    }

    // No block may leave while another still reads its partial tile.
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    if (ranks > 1) cluster_barrier();
    else __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_d), "r"(tmem_cols));
}

}  // namespace b200

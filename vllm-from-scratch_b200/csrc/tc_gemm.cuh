// y[M, I] = silu(x w_gate^T) * (x w_up^T) for many token rows (portions of prompts) on the
// 5th-generation tensor cores: the feed-forward's first product with its activation in the
// epilogue, so that the [M, 2 I] product is never written and read again.  w is [2 I, K] with I
// gate rows followed by I up rows; a tile holds matching halves of both.
//
// One persistent block per SM walks over tiles of 128 token rows x BN weight rows (BN / 2 gate
// rows and the BN / 2 up rows that belong to them).  Six warps:
//   0     one thread requests the copies: per 64 elements of K a [128 x 64] block of x and two
//         [BN / 2 x 64] blocks of w by tensor copies (TMA, 128-byte swizzle) into a ring of stages;
//   1     one thread issues the MMAs (tcgen05.mma, M 128, N BN, K 16; four per stage) into one of
//         two accumulators in tensor memory and hands each stage back with tcgen05.commit;
//   2-5   epilogue: a thread owns a token row (a lane of tensor memory), reads the finished
//         accumulator 32 gate and 32 up columns at a time and stores; meanwhile the MMAs of the
//         next tile fill the other accumulator.
// Tiles are numbered with the token-row block running fastest, so that the blocks at work at
// the same time share tiles of w (read from memory once) and x stays in L2.  Token rows past M
// read as zeros and are not stored.  Waits are bounded.
#pragma once

#include "tcgen05.cuh"

namespace b200 {

constexpr int kTgRows = 128;                    // token rows per tile = UMMA M
constexpr int kTgK = 64;                        // elements of K per stage
constexpr int kTgThreads = 6 * 32;
constexpr int kTgXBytes = kTgRows * kTgK * 2;   // 16 KB
constexpr int kTgSmemLimit = 220 * 1024;

template <int BN> struct TcGemmShape {
    static constexpr int kStageBytes = kTgXBytes + BN * kTgK * 2;
    static constexpr int kFit = (kTgSmemLimit - 2048) / kStageBytes;
    static constexpr int kStages = kFit > 6 ? 6 : kFit;
    static constexpr int kSmem = kStages * kStageBytes + 1024 + 1024;   // stages, barriers, room to align to 1024 bytes
};

template <int BN>
__global__ void __launch_bounds__(kTgThreads, 1) tc_gated_gemm_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    __nv_bfloat16* __restrict__ y, int M, int N, int K, int* __restrict__ error_flag) {
    // N: rows of each of the two halves of w (= columns of y).
    constexpr int kStages = TcGemmShape<BN>::kStages;
    constexpr int kStageBytes = TcGemmShape<BN>::kStageBytes;
    constexpr int kColumns = BN <= 128 ? 256 : 512;             // tensor memory for two accumulators: a power of two
    constexpr int kOut = BN / 2;                                // columns of y per tile
    extern __shared__ unsigned char tg_smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)tg_smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* full = reinterpret_cast<unsigned long long*>(smem + kStages * kStageBytes);
    unsigned long long* empty = full + kStages;
    unsigned long long* acc_full = empty + kStages;             // [2] the MMAs of a tile are complete
    unsigned long long* acc_empty = acc_full + 2;               // [2] the epilogue has read the accumulator
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    overlap_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_blocks = (M + kTgRows - 1) / kTgRows, n_blocks = N / kOut;
    const int tiles = m_blocks * n_blocks, k_blocks = K / kTgK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full + a, 1);
            mbar_init(acc_empty + a, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(kColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // -------- copies --------
        if (lane == 0) {
            overlap_wait();                                     // x comes from the kernel before this one
            int stage = 0;
            unsigned round = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_blocks) * kTgRows, n_block = tile / m_blocks;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty + stage, (round & 1u) ^ 1u)) {
                        atomicExch(error_flag, 51);
                        ok = false;
                        break;
                    }
                    unsigned char* x_tile = smem + stage * kStageBytes;
                    unsigned char* w_tile = x_tile + kTgXBytes;
                    mbar_expect_tx(full + stage, (unsigned)kStageBytes);
                    tma_load_2d(x_tile, &map_x, kb * kTgK, m0, full + stage);
                    tma_load_2d(w_tile, &map_w, kb * kTgK, n_block * (BN / 2), full + stage);
                    tma_load_2d(w_tile + (BN / 2) * 128, &map_w, kb * kTgK, N + n_block * (BN / 2), full + stage);
                    if (++stage == kStages) {
                        stage = 0;
                        ++round;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------- MMAs --------
        if (lane == 0) {
            const unsigned idesc = umma_idesc(BN);
            int stage = 0;
            unsigned round = 0;
            int count = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++count) {
                const int acc = count & 1;
                // the epilogue has read what the tile two back left in this accumulator
                if (!mbar_wait(acc_empty + acc, (((unsigned)count >> 1) & 1u) ^ 1u)) {
                    atomicExch(error_flag, 52);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_acc = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full + stage, round & 1u)) {
                        atomicExch(error_flag, 53);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* x_tile = smem + stage * kStageBytes;
                    const unsigned long long x_desc = umma_desc(x_tile, 0), w_desc = umma_desc(x_tile + kTgXBytes, 0);
#pragma unroll
                    for (int j = 0; j < kTgK / 16; ++j)             // 16 elements of K = 32 bytes further on in both tiles
                        umma_bf16(tmem_acc, x_desc + (unsigned long long)(j * 2), w_desc + (unsigned long long)(j * 2), idesc,
                                  kb > 0 || j > 0);
                    umma_commit(empty + stage);                   // the stage is free when these MMAs have read it
                    if (++stage == kStages) {
                        stage = 0;
                        ++round;
                    }
                }
                if (ok) umma_commit(acc_full + acc);
            }
        }
    } else {
        // -------- epilogue: a thread is a token row --------
        const int quarter = warp & 3;                           // the lanes of tensor memory this warp may touch
        const int row = quarter * 32 + lane;
        const unsigned lane_base = (unsigned)(quarter * 32) << 16;
        bool ok = true;
        int count = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++count) {
            const int m = (tile % m_blocks) * kTgRows + row, n_block = tile / m_blocks;
            const int acc = count & 1;
            if (ok && !mbar_wait(acc_full + acc, ((unsigned)count >> 1) & 1u)) {
                atomicExch(error_flag, 54);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned tmem_acc = tmem_base + lane_base + acc * BN;
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < kOut; c += 32) {
                    float gate[32], up[32];
                    tmem_ld32(tmem_acc + c, gate);
                    tmem_ld32(tmem_acc + BN / 2 + c, up);
                    unsigned packed[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        const __nv_bfloat162 pair = __floats2bfloat162_rn(gate[e] / (1.0f + __expf(-gate[e])) * up[e],
                                                                          gate[e + 1] / (1.0f + __expf(-gate[e + 1])) * up[e + 1]);
                        packed[e >> 1] = *reinterpret_cast<const unsigned*>(&pair);
                    }
                    if (m < M) {
                        uint4* dst = reinterpret_cast<uint4*>(y + (size_t)m * N + (size_t)n_block * kOut + c);
#pragma unroll
                        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                    }
                }
            }
            // the accumulator has been read: the MMAs of the tile after next may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(kColumns));
}

}  // namespace b200

// Paged causal attention for portions of prompts on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory), head size 128, bfloat16.
//
// One block = 256 consecutive query tokens of one request x one query head, as two
// groups of 128 rows that share every tile of keys and values.  Eleven warps:
//   0-7  softmax, four per group; a thread owns one query row, which is one lane of
//        tensor memory, so the softmax needs no exchange between threads;
//   8-9  one thread per group issues the group's MMAs;
//   10   requests the copies: lane j brings in page j of a tile (keys, then values),
//        four stages each, so that tiles arrive while the tiles before them are in use.
// Per tile of 64 keys and per group:
//   S = Q K^T       8 x tcgen05.mma (M 128, N 64, K 16), Q and K from shared memory
//                   (K-major, 128-byte swizzle, brought in by tensor copies page by page),
//                   into one of the group's two S buffers in tensor memory;
//   softmax         each thread reads its row of S (64 floats) from tensor memory once,
//                   keeps a reference exponent and the running sum in float32, and writes
//                   P as bfloat16 pairs back over the first 32 columns of the buffer.  The
//                   reference moves only when the row's maximum exceeds it by more than
//                   2^8; then the thread rescales its row of O in tensor memory.  (Any
//                   reference gives the same quotient O / sum; a stale one only shifts
//                   the exponent range of P, which bfloat16 has to spare.)
//   O += P V        4 x tcgen05.mma (M 128, N 128, K 16) with P read from tensor memory
//                   and V straight from its pages' layout ([key][channel], the "MN-major"
//                   operand form).
// With two S buffers a group's MMA thread issues S of tile t + 2 right after P V of tile t, so a
// group's next S is complete before its softmax asks for it: the softmax warps run tile
// after tile without waiting for the tensor pipe, and the two groups' MMAs fill each
// other's gaps.  The tensor pipe runs MMAs in the order of issue: S of tile t + 2
// overwrites P of tile t only after P V of tile t has read it.  O is rescaled only after
// the P V before it has finished (mbarriers of its own, one for even and one for odd tiles).  tcgen05.commit hands the stages of
// K and V back to the copying warp.
// Masking and arguments are those of attention_generic.cu.  Waits are bounded.
#pragma once

#include "tcgen05.cuh"

namespace b200 {

constexpr int kAtD = 128;                       // head size
constexpr int kAtRows = 128;                    // queries per block
constexpr int kAtKeys = 64;                     // keys per tile
constexpr int kAtHalf = kAtRows * 64 * 2;       // one [128 x 64] bfloat16 block: 16 KB

// Operands whose M/N index is the contiguous one ([k][mn] rows of 128 bytes, 128-byte swizzle)
// have their 64-wide blocks of the M/N index `lbo` bytes apart and groups of 8 k-rows 1024
// bytes apart.
//
// The MMA thread is one thread issuing dependent integer instructions: building a 64-bit
// descriptor for every MMA costs it more than the MMA costs the tensor pipe.  The upper
// word of all descriptors here is one constant (8-row groups 1024 bytes apart, version 1,
// 128-byte swizzle); the lower word is (address >> 4) plus the leading-offset field, so a
// tile's descriptors are one word per tile and one add per MMA.
constexpr unsigned kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ unsigned desc_lo_k_major(const void* smem_tile) {
    return ((smem_u32(smem_tile) & 0x3FFFF) >> 4) | (1u << 16);
}
__device__ __forceinline__ unsigned desc_lo_mn_major(const void* smem_tile, int lbo) {
    return ((smem_u32(smem_tile) & 0x3FFFF) >> 4) | ((unsigned)((lbo >> 4) & 0x3FFF) << 16);
}
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_ss(unsigned tmem_d, unsigned a_lo, unsigned b_lo, unsigned idesc) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\nsetp.ne.b32 p, %5, 0;\n"
        "mov.b64 da, {%1, %3};\nmov.b64 db, {%2, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n}\n" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "n"(ACCUMULATE ? 1 : 0)
        : "memory");
}
__device__ __forceinline__ void umma_ts(unsigned tmem_d, unsigned tmem_a, unsigned b_lo, unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 db;\nsetp.ne.b32 p, %5, 0;\n"
        "mov.b64 db, {%2, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 operations in one instruction (the packed forms of this architecture).
__device__ __forceinline__ float2 fma_pair(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add_pair(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// Issue the read of 32 columns into v[0..31]; the values are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(unsigned taddr, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
          "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]),
          "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]),
          "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_st32_bits(unsigned taddr, const unsigned* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}

// Shared memory (offsets from a 1024-byte aligned base): Q 2 x 32 KB, four stages of K and
// four of V (64 keys = 16 KB each), barriers.
constexpr int kAtStages = 4;
constexpr int kAtStageBytes = kAtKeys * kAtD * 2;           // 16 KB: two [64 x 64] blocks of 8 KB
constexpr int kAtStageHalf = kAtStageBytes / 2;
constexpr int kAtQ = 0, kAtK = 4 * kAtHalf, kAtV = kAtK + kAtStages * kAtStageBytes;
constexpr int kAtBars = kAtV + kAtStages * kAtStageBytes;
constexpr int kAtSmem = kAtBars + 512 + 1024;
constexpr int kAtGroups = 2;                    // 128-row groups per block
constexpr int kAtBlockRows = kAtGroups * kAtRows;
constexpr int kAtMmaWarp = 4 * kAtGroups, kAtCopyWarp = kAtMmaWarp + kAtGroups;   // one MMA warp per group
constexpr int kAtThreads = (kAtCopyWarp + 1) * 32;
constexpr float kAtRescaleStep = 8.0f;          // the reference exponent moves in steps larger than this

__global__ void __launch_bounds__(kAtThreads, 1) prefill_attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ query_start, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
    int num_requests, int max_pages, int nq, int nkv, int page_size, float scale_log2, int window,
    int token_offset, int key_splits, float* __restrict__ partial_o, float* __restrict__ partial_ml,
    int* __restrict__ error_flag) {
    // key_splits > 1 (grid.z): the block visits only its share of the row block's tiles of keys and
    // leaves O unnormalised, its reference exponent and its sum at
    // [(row of q * nq + head) * key_splits + blockIdx.z] of partial_o / partial_ml, for
    // merge_splits_kernel: few row blocks over many keys would leave most SMs idle otherwise.
    // token_offset: row of q and out at which the first of these requests begins (requests ahead of
    // them in the batch are another launch's); query_start holds rows of the whole batch.
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* q_bar = reinterpret_cast<unsigned long long*>(smem + kAtBars);
    unsigned long long* k_full = q_bar + 1;                 // [stages] keys of a stage have arrived
    unsigned long long* v_full = k_full + kAtStages;        // [stages] values of a stage have arrived
    unsigned long long* k_free = v_full + kAtStages;        // [stages] both groups' S MMAs have read the stage
    unsigned long long* v_free = k_free + kAtStages;        // [stages] both groups' P V MMAs have read the stage
    unsigned long long* s_bar = v_free + kAtStages;         // [group][buffer] S of a tile is in the buffer
    unsigned long long* p_bar = s_bar + 2 * kAtGroups;      // [group][buffer] all 128 rows of P are in the buffer
    unsigned long long* o_bar = p_bar + 2 * kAtGroups;      // [group][tile & 1] P V of the tile has been added to O
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(o_bar + 2 * kAtGroups);

    // Which request and which 256-row tile of it.  grid (query heads, tiles): blocks start in the
    // order of their index, x first, so the heaviest tiles of all heads start first, and the
    // heads that share keys and values run side by side.
    const int block = gridDim.y - 1 - blockIdx.y;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((query_start[mid] - token_offset) / kAtBlockRows + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int tile_first = (block - ((q_begin - token_offset) / kAtBlockRows + request)) * kAtBlockRows;
    if (tile_first >= q_len) return;
    const int rows_here = min(kAtBlockRows, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.x;
    const int kv_head = head / (nq / nkv);
    const int* table = block_table + (size_t)request * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int first_pos = past + tile_first;
    int k_first = window > 0 ? max(0, first_pos - window + 1) : 0;   // (moved on to this block's share below)
    k_first = (k_first / page_size) * page_size;
    k_first = (k_first / kAtKeys) * kAtKeys;                // pages larger than a tile: start on a tile's edge too
    // Tiles of 64 keys each group visits (a group without rows visits none).
    int group_tiles[kAtGroups];
#pragma unroll
    for (int g = 0; g < kAtGroups; ++g) {
        const int rows_g = min(kAtRows, rows_here - g * kAtRows);
        group_tiles[g] = rows_g > 0 ? (first_pos + g * kAtRows + rows_g - k_first + kAtKeys - 1) / kAtKeys : 0;
    }
    int tiles = max(group_tiles[0], group_tiles[1]);
    if (key_splits > 1) {
        // This block's share: tiles [begin, end) of the row block.  From here on the first key and
        // the tile counts are those of the share; nothing below knows of the others.
        const int share = (tiles + key_splits - 1) / key_splits;
        const int begin = min(tiles, (int)blockIdx.z * share), end = min(tiles, begin + share);
#pragma unroll
        for (int g = 0; g < kAtGroups; ++g) group_tiles[g] = max(0, min(group_tiles[g], end) - begin);
        tiles = end - begin;
        k_first += begin * kAtKeys;
    }
    const int copy_rows = min(page_size, kAtKeys);          // rows of one tensor copy (the tensor maps' box)
    const int copies_per_tile = kAtKeys / copy_rows;
    const int table_len = (seq_len + page_size - 1) / page_size;

    if (tid == 0) {
        mbar_init(q_bar, 1);
        for (int s = 0; s < kAtStages; ++s) {
            mbar_init(k_full + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(k_free + s, kAtGroups);
            mbar_init(v_free + s, kAtGroups);
        }
        for (int g = 0; g < kAtGroups; ++g) {
            mbar_init(s_bar + 2 * g, 1);
            mbar_init(s_bar + 2 * g + 1, 1);
            mbar_init(p_bar + 2 * g, kAtRows);
            mbar_init(p_bar + 2 * g + 1, kAtRows);
            mbar_init(o_bar + 2 * g, 1);
            mbar_init(o_bar + 2 * g + 1, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // Value rows that no copy fills (positions past the request's pages) must not hold
    // bit patterns of NaN: their probabilities are zero, and 0 x NaN would poison O.
    for (int i = tid; i < kAtStages * kAtStageBytes / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem + kAtV)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    // Tensor memory: group g has two S buffers of 64 columns at g * 128 (P over the first 32
    // columns of its buffer) and O at 256 + g * 128.
    const unsigned tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == kAtCopyWarp) {
        // -------- copies: lane j owns the j-th page (or part of a page) of every tile --------
        auto source_row = [&](int t) {          // first row of this lane's copy in the [pages x heads x page] x d matrix, or -1
            const int key = k_first + t * kAtKeys + lane * copy_rows;
            const int index = key / page_size;
            if (lane >= copies_per_tile || index >= table_len) return -1;
            const int page = table[index];
            return page < 0 ? -1 : (page * nkv + kv_head) * page_size + (key - index * page_size);
        };
        auto request_rows = [&](const CUtensorMap* map, unsigned char* stage, unsigned long long* bar, int row) {
            const unsigned valid = __ballot_sync(0xffffffffu, row >= 0);
            if (lane == 0) mbar_expect_tx(bar, (unsigned)__popc(valid) * copy_rows * kAtD * 2);
            __syncwarp();
            if (row >= 0) {
                unsigned char* dst = stage + lane * copy_rows * 128;
                tma_load_2d(dst, map, 0, row, bar);
                tma_load_2d(dst + kAtStageHalf, map, 64, row, bar);
            }
        };
        // Queries, keys and values come from the kernel ahead on the stream; everything up to here
        // (barriers, tensor memory, the zeroed stages) may have run beside its last blocks.  Nothing
        // else of this block reads or writes global memory before data that these copies bring.
        overlap_wait();
        if (lane == 0) {
            const int groups_here = rows_here > kAtRows ? 2 : 1;
            mbar_expect_tx(q_bar, (unsigned)groups_here * 2 * kAtHalf);
            for (int g = 0; g < groups_here; ++g) {
                tma_load_2d(smem + kAtQ + g * 2 * kAtHalf, &map_q, head * kAtD, q_begin + tile_first + g * kAtRows, q_bar);
                tma_load_2d(smem + kAtQ + g * 2 * kAtHalf + kAtHalf, &map_q, head * kAtD + 64,
                            q_begin + tile_first + g * kAtRows, q_bar);
            }
        }
        int next_row = source_row(0);
        for (int t = 0; t < tiles; ++t) {
            const int s = t % kAtStages, row = next_row;
            const unsigned freed = ((t / kAtStages) & 1) ^ 1;       // phase in which tile t - stages left the stage
            if (t + 1 < tiles) next_row = source_row(t + 1);
            if (t >= kAtStages && !mbar_wait(k_free + s, freed)) { atomicExch(error_flag, 21); ok = false; }
            if (!__all_sync(0xffffffffu, ok)) break;
            request_rows(&map_k, smem + kAtK + s * kAtStageBytes, k_full + s, row);
            if (t >= kAtStages && !mbar_wait(v_free + s, freed)) { atomicExch(error_flag, 22); ok = false; }
            if (!__all_sync(0xffffffffu, ok)) break;
            request_rows(&map_v, smem + kAtV + s * kAtStageBytes, v_full + s, row);
        }
    } else if (warp >= kAtMmaWarp) {
        // -------- per group, one thread issues the group's MMAs --------
        // The order is S(0), S(1), then for every tile t: P V(t), S(t + 2).  S(t + 2) goes
        // into the buffer that P(t) leaves, and the pipe runs it after P V(t) has read P(t).
        // A group's next S is therefore complete before its softmax asks for it, and the two
        // groups' MMAs fill each other's gaps.  A group past its last tile still takes part
        // in handing the stages back (the barriers count both groups).
        if (lane == 0) {
            const int g = warp - kAtMmaWarp;
            const int my_tiles = group_tiles[g];
            const unsigned idesc_s = umma_idesc(kAtKeys);                        // both operands K-major, N = 64
            const unsigned idesc_o = umma_idesc(kAtD) | (1u << 16);              // B (values) MN-major, N = 128
            const unsigned q_lo = desc_lo_k_major(smem + kAtQ + g * 2 * kAtHalf);
            const unsigned k_lo = desc_lo_k_major(smem + kAtK);
            const unsigned v_lo = desc_lo_mn_major(smem + kAtV, kAtStageHalf);
            const unsigned tmem_s0 = tmem_base + g * 2 * kAtKeys;
            const unsigned tmem_o = tmem_base + 2 * kAtGroups * kAtKeys + g * kAtD;
            auto issue_s = [&](int t) {                                          // S(t) = Q K(t)^T
                const int s = t % kAtStages;
                // (a group past its last tile waits too: it may hand a stage back once per filling)
                if (!mbar_wait(k_full + s, (t / kAtStages) & 1)) return false;
                if (t >= my_tiles) { mbar_arrive(k_free + s); return true; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned k_tile = k_lo + ((s * kAtStageBytes) >> 4);
                const unsigned tmem_s = tmem_s0 + (t & 1) * kAtKeys;
                // k-step j: 16 channels = 32 bytes inside a 64-channel block; blocks 16 KB (Q) and 8 KB (K) apart
                umma_ss<false>(tmem_s, q_lo, k_tile, idesc_s);
#pragma unroll
                for (int j = 1; j < kAtD / 16; ++j)
                    umma_ss<true>(tmem_s, q_lo + (((j >> 2) * kAtHalf + (j & 3) * 32) >> 4),
                                  k_tile + (((j >> 2) * kAtStageHalf + (j & 3) * 32) >> 4), idesc_s);
                umma_commit(s_bar + 2 * g + (t & 1));
                umma_commit(k_free + s);
                return true;
            };
            auto issue_o = [&](int t) {                                          // O += P(t) V(t)
                const int s = t % kAtStages;
                if (!mbar_wait(v_full + s, (t / kAtStages) & 1)) return false;
                if (t >= my_tiles) { mbar_arrive(v_free + s); return true; }
                if (!mbar_wait(p_bar + 2 * g + (t & 1), (t >> 1) & 1)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned v_tile = v_lo + ((s * kAtStageBytes) >> 4);
                const unsigned tmem_p = tmem_s0 + (t & 1) * kAtKeys;
                // k-step j: 16 keys = 8 columns of P, 16 rows of 128 bytes of V
#pragma unroll
                for (int j = 0; j < kAtKeys / 16; ++j)
                    umma_ts(tmem_o, tmem_p + j * 8, v_tile + ((j * 16 * 128) >> 4), idesc_o, t > 0 || j > 0);
                umma_commit(v_free + s);
                umma_commit(o_bar + 2 * g + (t & 1));
                return true;
            };
            ok = mbar_wait(q_bar, 0);
            for (int t = 0; t < 2 && t < tiles && ok; ++t) ok = issue_s(t);
            for (int t = 0; t < tiles && ok; ++t) {
                ok = issue_o(t);
                if (ok && t + 2 < tiles) ok = issue_s(t + 2);
            }
            if (!ok) atomicExch(error_flag, 23);
        }
    } else {
        // -------- softmax warps: a thread is a query row, which is a lane of tensor memory --------
        const int g = warp >> 2;
        const int row = (warp & 3) * 32 + lane;                 // row within the group
        const int my_tiles = group_tiles[g];
        const int q_pos = first_pos + g * kAtRows + row;
        const int warp_first = first_pos + g * kAtRows + (warp & 3) * 32, warp_last = warp_first + 31;
        const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
        const unsigned tmem_o = tmem_base + 2 * kAtGroups * kAtKeys + g * kAtD + lane_base;
        float row_ref = -INFINITY, row_sum = 0.0f;              // reference exponent, sum of exp2(s - reference)
        for (int t = 0; t < my_tiles; ++t) {
            const int k0 = k_first + t * kAtKeys;
            const int buffer = t & 1;
            const unsigned tmem_s = tmem_base + g * 2 * kAtKeys + buffer * kAtKeys + lane_base;
            if (ok && !mbar_wait(s_bar + 2 * g + buffer, (t >> 1) & 1)) { atomicExch(error_flag, 25); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // The row of S (64 values) in registers: one round trip to tensor memory.
            float sv[kAtKeys];
            tmem_ld32_issue(tmem_s, sv);
            tmem_ld32_issue(tmem_s + 32, sv + 32);
            tmem_ld_wait();
            // A tile wholly visible to every row of this warp (before its first query, inside
            // every window) needs no mask; only tiles on the diagonal or at a window's edge do.
            const bool all_visible = k0 + kAtKeys - 1 <= warp_first && (window <= 0 || k0 > warp_last - window);
            if (!all_visible) {
#pragma unroll
                for (int e = 0; e < kAtKeys; ++e) {
                    const int kp = k0 + e;
                    bool visible = kp <= q_pos;
                    if (window > 0) visible = visible && (kp > q_pos - window);
                    if (!visible) sv[e] = -INFINITY;
                }
            }
            // The exponentials are taken against the reference the row already has, which does
            // not wait for this tile's maximum; the maximum is found beside them (four chains),
            // and only a row whose maximum has outgrown the reference by more than 2^8, which
            // is rare after the first tiles, takes them again against the new one.
            // 64 keys become 32 columns of bfloat16 pairs (even key in the low half), written over S.
            unsigned packed[32];
            auto exponentials = [&](float ref) {
                const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-ref, -ref);
                float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float2 x = fma_pair(make_float2(sv[2 * e], sv[2 * e + 1]), scale2, shift2);
                    const float2 pr = make_float2(exp2_approx(x.x), exp2_approx(x.y));      // exp2(-inf) = 0
                    if (e & 1) sum_b = add_pair(sum_b, pr); else sum_a = add_pair(sum_a, pr);
                    const __nv_bfloat162 pair = __floats2bfloat162_rn(pr.x, pr.y);
                    packed[e] = *reinterpret_cast<const unsigned*>(&pair);
                }
                return (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
            };
            float tile_sum = exponentials(row_ref == -INFINITY ? 0.0f : row_ref);
            float max4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
            for (int e = 4; e < kAtKeys; ++e) max4[e & 3] = fmaxf(max4[e & 3], sv[e]);
            const float tile_max = fmaxf(fmaxf(max4[0], max4[1]), fmaxf(max4[2], max4[3])) * scale_log2;   // scale_log2 > 0
            const bool moved = tile_max > row_ref + kAtRescaleStep;          // also the first finite maximum
            float alpha = 1.0f;
            if (moved) {
                alpha = exp2_approx(row_ref - tile_max);                     // exp2(-inf) = 0
                row_ref = tile_max;
                tile_sum = exponentials(tile_max);
            }
            tmem_st32_bits(tmem_s, packed);
            row_sum = row_sum * alpha + tile_sum;
            // Rescale O where the reference moved (a whole warp at a time: the accesses are
            // collective), after the P V before this tile has finished.  That P V has its
            // barrier to itself until this thread's arrival below lets the next one be issued,
            // and "S of this tile is ready" implies that the P V two tiles back, the one before
            // on that barrier, is complete: the barrier is in the phase of the awaited P V or
            // one past it, so the parity wait is exact.
            if (t > 0 && ok && __any_sync(0xffffffffu, moved)) {
                if (!mbar_wait(o_bar + 2 * g + ((t - 1) & 1), ((t - 1) >> 1) & 1)) { atomicExch(error_flag, 27); ok = false; }
                ok = __all_sync(0xffffffffu, ok);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (ok) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float v[32];
                        tmem_ld32(tmem_o + c * 32, v);
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] *= alpha;
                        tmem_st32(tmem_o + c * 32, v);
                    }
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(p_bar + 2 * g + buffer);
        }

        // ---- O / sum to the output ----
        if (my_tiles > 0 && ok && !mbar_wait(o_bar + 2 * g + ((my_tiles - 1) & 1), ((my_tiles - 1) >> 1) & 1)) {
            atomicExch(error_flag, 26);
            ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
        const int row_in_block = g * kAtRows + row;
        __nv_bfloat16* dst = out + ((size_t)(q_begin + tile_first + row_in_block) * nq + head) * kAtD;
        if (key_splits > 1) {
            // (row_ref is -inf and row_sum 0 where the share held no tile for this group)
            const size_t slot = ((size_t)(q_begin + tile_first + row_in_block) * nq + head) * key_splits + blockIdx.z;
            float4* share_o = reinterpret_cast<float4*>(partial_o + slot * kAtD);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[32];
                if (my_tiles > 0 && ok) tmem_ld32(tmem_o + c * 32, v);
                else
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0.0f;
                if (row_in_block < rows_here && ok) {
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        share_o[c * 8 + q4] = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
                }
            }
            if (row_in_block < rows_here && ok) {
                partial_ml[slot * 2] = row_ref;
                partial_ml[slot * 2 + 1] = row_sum;
            }
        } else if (my_tiles > 0 && ok) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_ld32(tmem_o + c * 32, v);
                if (row_in_block < rows_here) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 packed;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[q4 * 8 + 0] * inv, v[q4 * 8 + 1] * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(v[q4 * 8 + 2] * inv, v[q4 * 8 + 3] * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q4 * 8 + 4] * inv, v[q4 * 8 + 5] * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(v[q4 * 8 + 6] * inv, v[q4 * 8 + 7] * inv);
                        packed.x = *reinterpret_cast<unsigned*>(&h0);
                        packed.y = *reinterpret_cast<unsigned*>(&h1);
                        packed.z = *reinterpret_cast<unsigned*>(&h2);
                        packed.w = *reinterpret_cast<unsigned*>(&h3);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = packed;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
}

}  // namespace b200

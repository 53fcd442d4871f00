// Paged causal attention for portions of prompts on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory), head size 128, bfloat16.
//
// One block = 256 consecutive query tokens of one request x one query head, as two
// groups of 128 rows.  Each group has four softmax warps; a thread owns one query row,
// which is one lane of tensor memory, so the softmax needs no exchange between threads,
// and the two groups share every tile of keys and values.  A ninth warp requests the
// copies and issues the MMAs.  Per tile of 128 keys and per group:
//   S = Q K^T       8 x tcgen05.mma (M 128, N 128, K 16), Q and K from shared memory
//                   (K-major, 128-byte swizzle, brought in by tensor copies page by page);
//   softmax         each thread reads its row of S from tensor memory twice (maximum,
//                   then exponentials), keeps running maximum and sum in float32,
//                   writes P as bfloat16 into shared memory in the operand layout and
//                   rescales its row of O in tensor memory when the maximum moved;
//   O += P V        8 x tcgen05.mma with V read straight from its pages' layout
//                   ([key][channel], i.e. the "MN-major" operand form).
// tcgen05.commit after each batch of MMAs arrives on an mbarrier (per group one for the S
// batches, one for the O batches); because the tensor pipe runs batches in order, "S of
// tile t is ready" also means "P V of tile t - 1 is done", which frees the P buffer, the
// V stage and O for rescaling.  Keys of tile t + 2 and values of tile t are requested when
// S of tile t is ready.
// Masking and arguments are those of attention_generic.cu.  Waits are bounded.
#pragma once

#include "tc_gemm.cuh"

namespace b200 {

constexpr int kAtD = 128;                       // head size
constexpr int kAtRows = 128;                    // queries per block
constexpr int kAtKeys = 128;                    // keys per tile
constexpr int kAtHalf = kAtRows * 64 * 2;       // one [128 x 64] bfloat16 block: 16 KB

// Matrix descriptor of an operand whose M/N index is the contiguous one ([k][mn] rows of
// 128 bytes, 128-byte swizzle): 64-wide blocks of the M/N index `lbo` bytes apart, groups
// of 8 k-rows 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc_mn(const void* smem_tile, int byte_offset, int lbo) {
    const unsigned address = (smem_u32(smem_tile) + byte_offset) & 0x3FFFF;
    unsigned long long desc = 0;
    desc |= (unsigned long long)(address >> 4);
    desc |= (unsigned long long)((lbo >> 4) & 0x3FFF) << 16;
    desc |= (unsigned long long)(1024 >> 4) << 32;
    desc |= (unsigned long long)1 << 46;
    desc |= (unsigned long long)2 << 61;
    return desc;
}

__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
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

// Shared memory (offsets from a 1024-byte aligned base): Q 2 x 32 KB, P 2 x 32 KB, two
// stages of K (32 KB each), one of V (32 KB), barriers.
constexpr int kAtQ = 0, kAtP = 4 * kAtHalf, kAtK = 8 * kAtHalf, kAtV = 12 * kAtHalf, kAtBars = 14 * kAtHalf;
constexpr int kAtSmem = kAtBars + 128 + 1024;
constexpr int kAtGroups = 2;                    // 128-row groups per block
constexpr int kAtBlockRows = kAtGroups * kAtRows;
constexpr int kAtThreads = (4 * kAtGroups + 1) * 32;

__global__ void __launch_bounds__(kAtThreads, 1) prefill_attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ query_start, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
    int num_requests, int max_pages, int nq, int nkv, int page_size, float scale_log2, int window,
    int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* q_bar = reinterpret_cast<unsigned long long*>(smem + kAtBars);
    unsigned long long* k_bar = q_bar + 1;          // [2] stages of keys
    unsigned long long* v_bar = k_bar + 2;          // the stage of values
    unsigned long long* s_bar = v_bar + 1;          // [2] per group, once per tile: S ready
    unsigned long long* o_bar = s_bar + 2;          // [2] per group, once per tile: O updated
    unsigned long long* p_bar = o_bar + 2;          // [2] per group, once per tile: all 128 rows of P written
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(p_bar + 2);

    // Which request and which 256-row tile of it (heaviest tiles first).
    const int block = gridDim.x - 1 - blockIdx.x;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (query_start[mid] / kAtBlockRows + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int tile_first = (block - (q_begin / kAtBlockRows + request)) * kAtBlockRows;
    if (tile_first >= q_len) return;
    const int rows_here = min(kAtBlockRows, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const int* table = block_table + (size_t)request * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int first_pos = past + tile_first;
    int k_first = window > 0 ? max(0, first_pos - window + 1) : 0;
    k_first = (k_first / page_size) * page_size;
    // Tiles of keys each group visits (a group without rows visits none).
    int group_tiles[kAtGroups];
#pragma unroll
    for (int g = 0; g < kAtGroups; ++g) {
        const int rows_g = min(kAtRows, rows_here - g * kAtRows);
        group_tiles[g] = rows_g > 0 ? (first_pos + g * kAtRows + rows_g - k_first + kAtKeys - 1) / kAtKeys : 0;
    }
    const int tiles = max(group_tiles[0], group_tiles[1]);
    const int pages_per_tile = kAtKeys / page_size;
    const int table_len = (seq_len + page_size - 1) / page_size;

    if (tid == 0) {
        mbar_init(q_bar, 1);
        mbar_init(k_bar, 1); mbar_init(k_bar + 1, 1);
        mbar_init(v_bar, 1);
        for (int g = 0; g < kAtGroups; ++g) {
            mbar_init(s_bar + g, 1);
            mbar_init(o_bar + g, 1);
            mbar_init(p_bar + g, kAtRows);
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
    for (int i = tid; i < 2 * kAtHalf / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem + kAtV)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;          // S of group g at columns g * 128, O at 256 + g * 128
    bool ok = true;
    float row_max = -INFINITY, row_sum = 0.0f;

    if (warp == 4 * kAtGroups) {
        // -------- control warp: one thread requests the copies and issues the MMAs --------
        if (lane == 0) {
            auto load_kv = [&](const CUtensorMap* map, unsigned char* stage, unsigned long long* bar, int t) {
                const int first_page = (k_first + t * kAtKeys) / page_size;
                int valid = 0;
                for (int j = 0; j < pages_per_tile; ++j)
                    if (first_page + j < table_len && table[first_page + j] >= 0) ++valid;
                mbar_expect_tx(bar, (unsigned)valid * page_size * kAtD * 2);
                for (int j = 0; j < pages_per_tile; ++j) {
                    if (first_page + j >= table_len) continue;
                    const int page = table[first_page + j];
                    if (page < 0) continue;
                    const int row = (page * nkv + kv_head) * page_size;
                    unsigned char* dst = stage + j * page_size * 128;
                    tma_load_2d(dst, map, 0, row, bar);
                    tma_load_2d(dst + kAtHalf, map, 64, row, bar);
                }
            };
            const unsigned idesc_s = umma_idesc(kAtKeys);                        // both operands K-major
            const unsigned idesc_o = umma_idesc(kAtD) | (1u << 16);              // B (values) MN-major
            const int groups_here = rows_here > kAtRows ? 2 : 1;
            mbar_expect_tx(q_bar, (unsigned)groups_here * 2 * kAtHalf);
            for (int g = 0; g < groups_here; ++g) {
                tma_load_2d(smem + kAtQ + g * 2 * kAtHalf, &map_q, head * kAtD, q_begin + tile_first + g * kAtRows, q_bar);
                tma_load_2d(smem + kAtQ + g * 2 * kAtHalf + kAtHalf, &map_q, head * kAtD + 64,
                            q_begin + tile_first + g * kAtRows, q_bar);
            }
            load_kv(&map_k, smem + kAtK, k_bar, 0);
            if (tiles > 1) load_kv(&map_k, smem + kAtK + 2 * kAtHalf, k_bar + 1, 1);
            for (int t = 0; t < tiles && ok; ++t) {
                const int s = t & 1;
                bool ready = mbar_wait(k_bar + s, (t >> 1) & 1);
                if (t == 0) ready = ready && mbar_wait(q_bar, 0);
                if (!ready) { atomicExch(error_flag, 21); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* k_tile = smem + kAtK + s * 2 * kAtHalf;
                for (int g = 0; g < kAtGroups; ++g) {
                    if (t >= group_tiles[g]) continue;
                    const unsigned char* q_tile = smem + kAtQ + g * 2 * kAtHalf;
#pragma unroll
                    for (int j = 0; j < kAtD / 16; ++j)
                        umma_bf16(tmem_base + g * kAtKeys, umma_desc(q_tile + (j >> 2) * kAtHalf, (j & 3) * 32),
                                  umma_desc(k_tile + (j >> 2) * kAtHalf, (j & 3) * 32), idesc_s, j > 0);
                    umma_commit(s_bar + g);
                }
                // S of tile t ready means P V of tile t - 1 is done: the stage of V and stage s of K are free.
                for (int g = 0; g < kAtGroups; ++g)
                    if (t < group_tiles[g] && !mbar_wait(s_bar + g, t & 1)) { atomicExch(error_flag, 22); ok = false; }
                if (!ok) break;
                load_kv(&map_v, smem + kAtV, v_bar, t);
                if (t + 2 < tiles) load_kv(&map_k, smem + kAtK + s * 2 * kAtHalf, k_bar + s, t + 2);
                if (!mbar_wait(v_bar, t & 1)) { atomicExch(error_flag, 23); ok = false; break; }
                for (int g = 0; g < kAtGroups; ++g) {
                    if (t >= group_tiles[g]) continue;
                    if (!mbar_wait(p_bar + g, t & 1)) { atomicExch(error_flag, 24); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* p_tile = smem + kAtP + g * 2 * kAtHalf;
#pragma unroll
                    for (int j = 0; j < kAtKeys / 16; ++j)
                        umma_bf16(tmem_base + 2 * kAtKeys + g * kAtD, umma_desc(p_tile + (j >> 2) * kAtHalf, (j & 3) * 32),
                                  umma_desc_mn(smem + kAtV, j * 16 * 128, kAtHalf), idesc_o, t > 0 || j > 0);
                    umma_commit(o_bar + g);
                }
            }
        }
    } else {
        // -------- softmax warps: a thread is a query row, which is a lane of tensor memory --------
        const int g = warp >> 2;
        const int row = (warp & 3) * 32 + lane;                 // row within the group
        const int my_tiles = group_tiles[g];
        const int q_pos = first_pos + g * kAtRows + row;
        const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
        const unsigned tmem_s = tmem_base + g * kAtKeys, tmem_o = tmem_base + 2 * kAtKeys + g * kAtD;
        unsigned char* p_row = smem + kAtP + g * 2 * kAtHalf + (row >> 3) * 1024 + (row & 7) * 128;
        for (int t = 0; t < my_tiles; ++t) {
            const int k0 = k_first + t * kAtKeys;
            if (ok && !mbar_wait(s_bar + g, t & 1)) { atomicExch(error_flag, 25); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // pass 1: the row's maximum
            float tile_max = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_ld32(tmem_s + lane_base + c * 32, v);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int kp = k0 + c * 32 + e;
                    bool visible = kp <= q_pos;
                    if (window > 0) visible = visible && (kp > q_pos - window);
                    if (visible) tile_max = fmaxf(tile_max, v[e] * scale_log2);
                }
            }
            const float new_max = fmaxf(row_max, tile_max);
            const float ref = new_max == -INFINITY ? 0.0f : new_max;
            const float alpha = exp2f(row_max - ref);
            row_max = new_max;
            // pass 2: exponentials, their sum, P in the operand layout
            float tile_sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_ld32(tmem_s + lane_base + c * 32, v);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int kp = k0 + c * 32 + e;
                    bool visible = kp <= q_pos;
                    if (window > 0) visible = visible && (kp > q_pos - window);
                    v[e] = visible ? exp2f(v[e] * scale_log2 - ref) : 0.0f;
                    tile_sum += v[e];
                }
                // 32 keys = 4 chunks of 16 bytes; keys c*32.. lie in block (c >> 1), chunks (c & 1) * 4 ..
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c & 1) * 4 + q4;
                    uint4 packed;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v[q4 * 8 + 0], v[q4 * 8 + 1]);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(v[q4 * 8 + 2], v[q4 * 8 + 3]);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q4 * 8 + 4], v[q4 * 8 + 5]);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(v[q4 * 8 + 6], v[q4 * 8 + 7]);
                    packed.x = *reinterpret_cast<unsigned*>(&h0);
                    packed.y = *reinterpret_cast<unsigned*>(&h1);
                    packed.z = *reinterpret_cast<unsigned*>(&h2);
                    packed.w = *reinterpret_cast<unsigned*>(&h3);
                    *reinterpret_cast<uint4*>(p_row + (c >> 1) * kAtHalf + ((chunk ^ (row & 7)) << 4)) = packed;
                }
            }
            row_sum = row_sum * alpha + tile_sum;
            // rescale O where the maximum moved (a whole warp at a time: the accesses are collective)
            if (t > 0 && ok && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float v[32];
                    tmem_ld32(tmem_o + lane_base + c * 32, v);
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] *= alpha;
                    tmem_st32(tmem_o + lane_base + c * 32, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(p_bar + g);
        }

        // ---- O / sum to the output ----
        if (my_tiles > 0 && !mbar_wait(o_bar + g, (my_tiles - 1) & 1)) { atomicExch(error_flag, 26); ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
        const int row_in_block = g * kAtRows + row;
        __nv_bfloat16* dst = out + ((size_t)(q_begin + tile_first + row_in_block) * nq + head) * kAtD;
        if (my_tiles > 0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float v[32];
                tmem_ld32(tmem_o + lane_base + c * 32, v);
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

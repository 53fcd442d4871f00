// Paged causal attention for portions of prompts on the 5th-generation tensor cores
// (tcgen05, accumulators in tensor memory), head size 128, bfloat16.
//
// One block = 128 consecutive query tokens of one request x one query head; thread i
// owns query row i, which is lane i of tensor memory, so the softmax needs no
// exchange between threads.  Per tile of 128 keys:
//   S = Q K^T       8 x tcgen05.mma (M 128, N 128, K 16), Q and K from shared memory
//                   (K-major, 128-byte swizzle, brought in by tensor copies page by page);
//   softmax         each thread reads its row of S from tensor memory twice (maximum,
//                   then exponentials), keeps running maximum and sum in float32,
//                   writes P as bfloat16 into shared memory in the operand layout and
//                   rescales its row of O in tensor memory when the maximum moved;
//   O += P V        8 x tcgen05.mma with V read straight from its pages' layout
//                   ([key][channel], i.e. the "MN-major" operand form).
// tcgen05.commit after each batch of MMAs arrives on an mbarrier (one for the S batches,
// one for the O batches); because the tensor pipe runs batches in order, "S of tile t is
// ready" also means "P V of tile t - 1 is done", which frees the P buffer, the V stage
// and O for rescaling.
// Keys and values of tile t + 2 / t + 1 are requested while tile t is processed.
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

// Shared memory (offsets from a 1024-byte aligned base): Q 32 KB, P 32 KB, two stages of
// K (32 KB each) and of V (32 KB each), barriers.
constexpr int kAtQ = 0, kAtP = 2 * kAtHalf, kAtK = 4 * kAtHalf, kAtV = 8 * kAtHalf, kAtBars = 12 * kAtHalf;
constexpr int kAtSmem = kAtBars + 128 + 1024;

constexpr int kAtThreads = 160;                 // four softmax warps + one control warp

__global__ void __launch_bounds__(kAtThreads, 1) prefill_attention_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
    const int* __restrict__ query_start, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
    int num_requests, int max_pages, int nq, int nkv, int page_size, float scale_log2, int window,
    int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned long long* q_bar = reinterpret_cast<unsigned long long*>(smem + kAtBars);
    unsigned long long* k_bar = q_bar + 1;          // [2]
    unsigned long long* v_bar = k_bar + 2;          // [2]
    unsigned long long* s_bar = v_bar + 2;          // completes once per tile: S ready
    unsigned long long* o_bar = s_bar + 1;          // completes once per tile: O updated
    unsigned long long* p_bar = o_bar + 1;          // completes once per tile: all 128 rows of P written
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(p_bar + 1);

    // Which request and which 128-row tile of it (heaviest tiles first).
    const int block = gridDim.x - 1 - blockIdx.x;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (query_start[mid] / kAtRows + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int tile_first = (block - (q_begin / kAtRows + request)) * kAtRows;
    if (tile_first >= q_len) return;
    const int rows_here = min(kAtRows, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const int* table = block_table + (size_t)request * max_pages;
    const int tid = threadIdx.x, warp = tid >> 5;

    const int first_pos = past + tile_first;
    const int last_pos = first_pos + rows_here - 1;
    int k_first = window > 0 ? max(0, first_pos - window + 1) : 0;
    k_first = (k_first / page_size) * page_size;
    const int k_end = last_pos + 1;
    const int tiles = (k_end - k_first + kAtKeys - 1) / kAtKeys;
    const int pages_per_tile = kAtKeys / page_size;
    const int table_len = (seq_len + page_size - 1) / page_size;

    if (tid == 0) {
        mbar_init(q_bar, 1);
        mbar_init(k_bar, 1); mbar_init(k_bar + 1, 1);
        mbar_init(v_bar, 1); mbar_init(v_bar + 1, 1);
        mbar_init(s_bar, 1);
        mbar_init(o_bar, 1);
        mbar_init(p_bar, kAtRows);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // Value rows that no copy fills (positions past the request's pages) must not hold
    // bit patterns of NaN: their probabilities are zero, and 0 x NaN would poison O.
    for (int i = tid; i < 4 * kAtHalf / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem + kAtV)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_s = *tmem_slot, tmem_o = tmem_s + kAtKeys;
    bool ok = true;

    // ---- copies, issued by thread 0 ----
    auto load_k = [&](int t) {
        const int s = t & 1;
        const int first_page = (k_first + t * kAtKeys) / page_size;
        int valid = 0;
        for (int j = 0; j < pages_per_tile; ++j)
            if (first_page + j < table_len && table[first_page + j] >= 0) ++valid;
        mbar_expect_tx(k_bar + s, (unsigned)valid * page_size * kAtD * 2);
        for (int j = 0; j < pages_per_tile; ++j) {
            if (first_page + j >= table_len) continue;
            const int page = table[first_page + j];
            if (page < 0) continue;
            const int row = (page * nkv + kv_head) * page_size;
            unsigned char* dst = smem + kAtK + s * 2 * kAtHalf + j * page_size * 128;
            tma_load_2d(dst, &map_k, 0, row, k_bar + s);
            tma_load_2d(dst + kAtHalf, &map_k, 64, row, k_bar + s);
        }
    };
    auto load_v = [&](int t) {
        const int s = t & 1;
        const int first_page = (k_first + t * kAtKeys) / page_size;
        int valid = 0;
        for (int j = 0; j < pages_per_tile; ++j)
            if (first_page + j < table_len && table[first_page + j] >= 0) ++valid;
        mbar_expect_tx(v_bar + s, (unsigned)valid * page_size * kAtD * 2);
        for (int j = 0; j < pages_per_tile; ++j) {
            if (first_page + j >= table_len) continue;
            const int page = table[first_page + j];
            if (page < 0) continue;
            const int row = (page * nkv + kv_head) * page_size;
            unsigned char* dst = smem + kAtV + s * 2 * kAtHalf + j * page_size * 128;
            tma_load_2d(dst, &map_v, 0, row, v_bar + s);
            tma_load_2d(dst + kAtHalf, &map_v, 64, row, v_bar + s);
        }
    };
    float row_max = -INFINITY, row_sum = 0.0f;
    const unsigned idesc_s = umma_idesc(kAtKeys);                        // both operands K-major
    const unsigned idesc_o = umma_idesc(kAtD) | (1u << 16);              // B (values) MN-major

    if (warp == 4) {
        // -------- control warp: one thread requests the copies and issues the MMAs --------
        if (tid == 128) {
            mbar_expect_tx(q_bar, 2 * kAtHalf);
            tma_load_2d(smem + kAtQ, &map_q, head * kAtD, q_begin + tile_first, q_bar);
            tma_load_2d(smem + kAtQ + kAtHalf, &map_q, head * kAtD + 64, q_begin + tile_first, q_bar);
            load_k(0);
            load_v(0);
            if (tiles > 1) load_k(1);
            for (int t = 0; t < tiles && ok; ++t) {
                const int s = t & 1;
                bool ready = mbar_wait(k_bar + s, (t >> 1) & 1);
                if (t == 0) ready = ready && mbar_wait(q_bar, 0);
                if (!ready) { atomicExch(error_flag, 21); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* k_tile = smem + kAtK + s * 2 * kAtHalf;
#pragma unroll
                for (int j = 0; j < kAtD / 16; ++j)
                    umma_bf16(tmem_s, umma_desc(smem + kAtQ + (j >> 2) * kAtHalf, (j & 3) * 32),
                              umma_desc(k_tile + (j >> 2) * kAtHalf, (j & 3) * 32), idesc_s, j > 0);
                umma_commit(s_bar);
                // When S of tile t is ready, P V of tile t - 1 is done as well: stage s of K and
                // the other stage of V are free for the tiles to come.
                if (!mbar_wait(s_bar, t & 1)) { atomicExch(error_flag, 22); ok = false; break; }
                if (t + 2 < tiles) load_k(t + 2);
                if (t + 1 < tiles) load_v(t + 1);
                if (!mbar_wait(p_bar, t & 1) || !mbar_wait(v_bar + s, (t >> 1) & 1)) {
                    atomicExch(error_flag, 23);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* v_tile = smem + kAtV + s * 2 * kAtHalf;
#pragma unroll
                for (int j = 0; j < kAtKeys / 16; ++j)
                    umma_bf16(tmem_o, umma_desc(smem + kAtP + (j >> 2) * kAtHalf, (j & 3) * 32),
                              umma_desc_mn(v_tile, j * 16 * 128, kAtHalf), idesc_o, t > 0 || j > 0);
                umma_commit(o_bar);
            }
        }
    } else {
        // -------- softmax warps: thread = query row = lane of tensor memory --------
        const int row = tid;
        const int q_pos = first_pos + row;
        const unsigned lane_base = (unsigned)(warp * 32) << 16;
        unsigned char* p_row = smem + kAtP + (row >> 3) * 1024 + (row & 7) * 128;
        for (int t = 0; t < tiles; ++t) {
            const int k0 = k_first + t * kAtKeys;
            if (ok && !mbar_wait(s_bar, t & 1)) { atomicExch(error_flag, 24); ok = false; }
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
            mbar_arrive(p_bar);
        }
    }

    // ---- O / sum to the output ----
    if (warp < 4) {
    const int row = tid;
    const unsigned lane_base = (unsigned)(warp * 32) << 16;
    if (tiles > 0 && !mbar_wait(o_bar, (tiles - 1) & 1)) { atomicExch(error_flag, 25); ok = false; }
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;
    __nv_bfloat16* dst = out + ((size_t)(q_begin + tile_first + row) * nq + head) * kAtD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float v[32];
        if (tiles > 0) tmem_ld32(tmem_o + lane_base + c * 32, v);
        else
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0.0f;
        if (row < rows_here) {
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
    (void)ok;
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_s), "r"(256));
}

}  // namespace b200

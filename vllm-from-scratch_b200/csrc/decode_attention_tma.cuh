// Decode attention (one query token per request, keys split over blocks) with the keys
// and values brought in by tensor copies (TMA) instead of per-thread 16-byte copies.
//
// The arithmetic is that of decode_attention_kernel (attention_bf16_kernels.cuh): the
// query heads that share a key/value head are the rows of a 16-row fragment, a tile is
// 64 keys, each of four warps takes 16 of them through m16n8k16 products, softmax
// statistics in float32, partial (maximum, sum, output) per split.  What differs is how a
// tile gets into shared memory: a fifth warp requests it, lane j one copy of
// min(page, 64) rows x 64 channels per channel block, straight from the page, with the
// hardware's 128-byte swizzle; an mbarrier per stage counts the bytes in, another the
// four warps out.  The compute warps execute no address arithmetic and no copy
// instructions, which is where the other kernel spends most of its issue slots.
//
// Tiles start at multiples of 64 keys from a 64-aligned first key, so a window's first
// key may lie inside the first tile: keys before it are masked like keys past the end.
// Rows that no copy fills (past the end, pages given back) keep what the stage held;
// the value stages are zeroed once so that this is never a NaN pattern.
// grid (splits, kv heads, requests), 160 threads.  Waits are bounded.
//
// FUSED: the kernel takes the packed projection [T, (nq + 2 nkv) d] itself and does what
// head_norm_rope_cache_kernel (rope_cache.cu) does for a decode step, with its arithmetic:
// every block normalises and rotates the query heads of its group into shared memory; the
// block whose keys end at the newest position also normalises and rotates the new key,
// writes it and the new value into their page, and puts both into the row of its last tile
// that the copy of the page filled with what the slot held before.  A step then has one
// kernel less in its chain, and no tile has to wait for the kernel ahead: all of them come
// from earlier steps.
#pragma once

#include "attention_bf16_kernels.cuh"
#include "tcgen05.cuh"

namespace b200 {

constexpr int kDtStages = 2;
constexpr int kDtThreads = 160;                 // four compute warps and the copying warp

// What the fused form needs beside the attention's own arguments (see rope_cache.cu).
struct DecodeRope {
    const int* positions;       // [T]
    const int* slots;           // [T] page * page_size + offset of the new key, negative: do not store
    const float* q_weight;      // [d] or null: no norm
    const float* k_weight;
    const float* inv_freq;      // [d / 2]
    bf16* k_pages;
    bf16* v_pages;
    float eps;
};
template <int D> constexpr int decode_rope_smem() { return D * 4 + 16 * D * 2 + 2 * D * 2; }   // sin, cos; q; new key, value

template <int D, bool FUSED>
__global__ void __launch_bounds__(kDtThreads, D <= 128 ? 3 : 1) decode_attention_tma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ partial_o,
    float* __restrict__ partial_ml, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
    int max_pages, int nq, int nkv, int page_size, float scale_log2, int window, int splits,
    int* __restrict__ error_flag, DecodeRope rope) {
    static_assert(!FUSED || D == 128, "the fused form holds two pairs of channels per lane");
    constexpr int kBlocks = D / 64;                         // channel blocks of 64 (128 bytes a row)
    constexpr int kBlockBytes = kKeys * 128;                // one [64 keys x 64 channels] block
    constexpr int kTileBytes = kBlocks * kBlockBytes;       // K or V of a tile
    extern __shared__ unsigned char smem_dt[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dt + 1023) & ~(uintptr_t)1023);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + kDtStages * 2 * kTileBytes);
    unsigned long long* empty_bar = full_bar + kDtStages;
    float* sin_s = reinterpret_cast<float*>(smem + kDtStages * 2 * kTileBytes + 64);     // FUSED only, [D / 2] each
    float* cos_s = sin_s + D / 2;
    bf16* q_s = reinterpret_cast<bf16*>(cos_s + D / 2);                                 // [16][D]
    bf16* new_s = q_s + 16 * D;                                                         // [2][D]: new key, new value
    overlap_trigger();
    const int split = blockIdx.x, kv_head = blockIdx.y, request = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = nq / nkv;
    const int seq_len = seq_lens[request];
    const int k_lo = window > 0 ? max(0, seq_len - window) : 0;         // first visible key
    const int k_first = (k_lo / kKeys) * kKeys;
    const int total = seq_len - k_first;
    int chunk = (total + splits - 1) / splits;
    chunk = ((chunk + kKeys - 1) / kKeys) * kKeys;
    const int my_begin = k_first + split * chunk;
    const int my_end = min(seq_len, my_begin + chunk);
    const int tiles = my_end > my_begin ? (my_end - my_begin + kKeys - 1) / kKeys : 0;
    const int* table = block_table + (size_t)request * max_pages;
    const bool owner = FUSED && tiles > 0 && my_end == seq_len;         // this block's keys end at the newest one

    if (tid == 0) {
        for (int s = 0; s < kDtStages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // Value rows that no copy will fill must not hold NaN patterns (their probabilities are
    // zero, and 0 x NaN would poison the output).  Without a window every tile but the last
    // is filled whole and the last from its first row on: only the rows after its last copy
    // can stay as they were.  With a window pages may be missing anywhere: zero everything.
    {
        const int copy_rows = min(page_size, kKeys);
        const int last_keys = tiles > 0 ? (my_end - my_begin) - (tiles - 1) * kKeys : kKeys;
        const int first_unfilled = window > 0 ? 0 : min(kKeys, (last_keys + copy_rows - 1) / copy_rows * copy_rows);
        const int rows = kKeys - first_unfilled;                    // per channel block and stage
        for (int i = tid; i < kDtStages * kBlocks * rows * 8; i += kDtThreads) {
            const int chunk = i & 7, row = first_unfilled + (i >> 3) % rows, block = (i >> 3) / rows;   // block over stages too
            const int s = block / kBlocks, b = block - s * kBlocks;
            reinterpret_cast<uint4*>(smem + (s * 2 + 1) * kTileBytes + b * kBlockBytes + row * 128)[chunk] = make_uint4(0, 0, 0, 0);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncthreads();
    // Only the newest key and value (and the queries) come from the kernel before this one:
    // tiles that end before the newest position are requested before waiting for it.  (FUSED:
    // the kernel makes the newest key and value itself, so no tile waits; block tables,
    // lengths, positions and slots are inputs of the step, in place before its first kernel.)
    bool ok = true;

    float o[D / 8][4];
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    const int row_a = lane >> 2, row_b = row_a + 8;

    if (warp == 4) {
        // -------- copies: lane j owns the j-th page (or part of a page) of every tile --------
        const int copy_rows = min(page_size, kKeys);
        const int copies_per_tile = kKeys / copy_rows;
        const int table_len = (seq_len + page_size - 1) / page_size;
        bool waited = false;
        for (int t = 0; t < tiles; ++t) {
            const int s = t % kDtStages;
            if (!FUSED && !waited && (t >= kDtStages || my_begin + (t + 1) * kKeys >= seq_len)) {
                overlap_wait();
                waited = true;
            }
            const int key = my_begin + t * kKeys + lane * copy_rows;
            const int index = key / page_size;
            int row = -1;
            if (lane < copies_per_tile && key < my_end && index < table_len) {
                const int page = table[index];
                if (page >= 0) row = (page * nkv + kv_head) * page_size + (key - index * page_size);
            }
            if (t >= kDtStages && !mbar_wait(empty_bar + s, ((t / kDtStages) & 1) ^ 1)) { atomicExch(error_flag, 31); ok = false; }
            if (!__all_sync(0xffffffffu, ok)) break;
            const unsigned valid = __ballot_sync(0xffffffffu, row >= 0);
            if (lane == 0) mbar_expect_tx(full_bar + s, (unsigned)__popc(valid) * copy_rows * D * 2 * 2);
            __syncwarp();
            if (row >= 0) {
                unsigned char* k_dst = smem + (s * 2) * kTileBytes + lane * copy_rows * 128;
                unsigned char* v_dst = k_dst + kTileBytes;
#pragma unroll
                for (int b = 0; b < kBlocks; ++b) {
                    tma_load_2d(k_dst + b * kBlockBytes, &map_k, b * 64, row, full_bar + s);
                    tma_load_2d(v_dst + b * kBlockBytes, &map_v, b * 64, row, full_bar + s);
                }
            }
        }
    } else {
        // -------- four warps, 16 keys of every tile each --------
        unsigned qa[D / 16][4];
        if (FUSED) {
            // Before the wait: what does not come from the kernel ahead (position, angles, weights, slot).
            const float pos = (float)rope.positions[request];
            if (tid < D / 2) sincosf(pos * rope.inv_freq[tid], &sin_s[tid], &cos_s[tid]);
            const int slot = rope.slots[request];
            float qw1[2], qw2[2], kw1[2], kw2[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int j = lane + 32 * i;
                qw1[i] = rope.q_weight ? rope.q_weight[j] : 1.0f;
                qw2[i] = rope.q_weight ? rope.q_weight[j + D / 2] : 1.0f;
                kw1[i] = rope.k_weight ? rope.k_weight[j] : 1.0f;
                kw2[i] = rope.k_weight ? rope.k_weight[j + D / 2] : 1.0f;
            }
            asm volatile("bar.sync 2, 128;\n" ::: "memory");          // the angles are in shared memory
            overlap_wait();
            const int total_heads = nq + 2 * nkv;
            const bf16* row = q + (size_t)request * total_heads * D;            // q is the packed projection here
            const int items = group + (owner ? 2 : 0);                          // query heads, new key, new value
            for (int item = warp; item < items; item += 4) {
                const bool is_q = item < group, is_k = item == group;
                const int head = is_q ? kv_head * group + item : (is_k ? nq + kv_head : nq + nkv + kv_head);
                const bf16* src = row + (size_t)head * D;
                bf16* stored = nullptr;                                         // the new key's or value's place in its page
                if (!is_q && slot >= 0) {
                    const int page = slot / page_size, offset = slot - page * page_size;
                    stored = (is_k ? rope.k_pages : rope.v_pages) + (((size_t)page * nkv + kv_head) * page_size + offset) * D;
                }
                bf16 held[4];                                                   // channels lane, lane + 32, + 64, + 96
#pragma unroll
                for (int i = 0; i < 4; ++i) held[i] = src[lane + 32 * i];
                if (!is_q && !is_k) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        new_s[D + lane + 32 * i] = held[i];
                        if (stored) stored[lane + 32 * i] = held[i];
                    }
                    continue;
                }
                const float* weight = is_q ? rope.q_weight : rope.k_weight;
                float inv = 1.0f;
                if (weight) {
                    float sum_sq = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {                               // the order of rope_cache.cu's loop
                        const float v = to_float(held[i]);
                        sum_sq = fmaf(v, v, sum_sq);
                    }
                    sum_sq = warp_sum(sum_sq);
                    inv = rsqrtf(sum_sq / (float)D + rope.eps);
                }
                bf16* dst = is_q ? q_s + item * D : new_s;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j = lane + 32 * i;
                    const float x1 = to_float(held[i]) * inv * (is_q ? qw1[i] : kw1[i]);
                    const float x2 = to_float(held[i + 2]) * inv * (is_q ? qw2[i] : kw2[i]);
                    float r1, r2;
                    rotate_pair(x1, x2, cos_s[j], sin_s[j], r1, r2);
                    const bf16 o1 = from_float<bf16>(r1), o2 = from_float<bf16>(r2);
                    dst[j] = o1;
                    dst[j + D / 2] = o2;
                    if (stored) {
                        stored[j] = o1;
                        stored[j + D / 2] = o2;
                    }
                }
            }
            asm volatile("bar.sync 2, 128;\n" ::: "memory");          // queries and the new key and value are in shared memory
            load_q_fragments<D>(qa, row_a < group ? q_s + row_a * D : nullptr, row_b < group ? q_s + row_b * D : nullptr,
                                lane);
        } else {
            overlap_wait();
            const bf16* q_base = q + ((size_t)request * nq + (size_t)kv_head * group) * D;
            load_q_fragments<D>(qa, row_a < group ? q_base + (size_t)row_a * D : nullptr,
                                row_b < group ? q_base + (size_t)row_b * D : nullptr, lane);
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
        const int mi = lane >> 3, ri = lane & 7;
        for (int t = 0; t < tiles; ++t) {
            const int s = t % kDtStages;
            const int k0 = my_begin + t * kKeys;
            if (ok && !mbar_wait(full_bar + s, (t / kDtStages) & 1)) { atomicExch(error_flag, 32); ok = false; }
            ok = __all_sync(0xffffffffu, ok);
            const unsigned char* k_s = smem + (s * 2) * kTileBytes;
            const unsigned char* v_s = k_s + kTileBytes;
            if (FUSED && owner && t == tiles - 1) {
                // The newest key's row holds what its slot held before this step: the warp whose
                // 16 keys include it (no other warp reads the row) puts the new key and value there.
                const int r = seq_len - 1 - k0;
                if ((r >> 4) == warp) {
                    const int c = lane & 15;                                    // 16-byte chunk of the row
                    const uint4 fresh = reinterpret_cast<const uint4*>(new_s + (lane >= 16 ? D : 0))[c];
                    unsigned char* tile = smem + (s * 2 + (lane >= 16 ? 1 : 0)) * kTileBytes;
                    *reinterpret_cast<uint4*>(tile + (c >> 3) * kBlockBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = fresh;
                    __syncwarp();
                }
            }

            // scores of this warp's 16 keys
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int key = warp * 16 + (mi >> 1) * 8 + ri;
                const int chunk_k = ks * 2 + (mi & 1);               // 16-byte chunk of the row
                unsigned b[4];
                ldmatrix_x4(b, k_s + (chunk_k >> 3) * kBlockBytes + key * 128 + (((chunk_k & 7) ^ (key & 7)) << 4));
                mma_bf16(sc[0], qa[ks], b[0], b[1]);
                mma_bf16(sc[1], qa[ks], b[2], b[3]);
            }
            float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kp = k0 + warp * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = (kp >= k_lo && kp < my_end) ? sc[nt][e] * scale_log2 : -INFINITY;
                    sc[nt][e] = v;
                    if (e < 2) max_a = fmaxf(max_a, v); else max_b = fmaxf(max_b, v);
                }
            max_a = quad_max(max_a);
            max_b = quad_max(max_b);
            const float new_a = fmaxf(m_a, max_a), new_b = fmaxf(m_b, max_b);
            const float ref_a = new_a == -INFINITY ? 0.0f : new_a, ref_b = new_b == -INFINITY ? 0.0f : new_b;
            const float alpha_a = exp2f(m_a - ref_a), alpha_b = exp2f(m_b - ref_b);
            m_a = new_a;
            m_b = new_b;
            float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                sc[nt][0] = exp2f(sc[nt][0] - ref_a);
                sc[nt][1] = exp2f(sc[nt][1] - ref_a);
                sc[nt][2] = exp2f(sc[nt][2] - ref_b);
                sc[nt][3] = exp2f(sc[nt][3] - ref_b);
                sum_a += sc[nt][0] + sc[nt][1];
                sum_b += sc[nt][2] + sc[nt][3];
            }
            l_a = l_a * alpha_a + sum_a;
            l_b = l_b * alpha_b + sum_b;
            unsigned pa[4] = {pack_bf16(sc[0][0], sc[0][1]), pack_bf16(sc[0][2], sc[0][3]),
                              pack_bf16(sc[1][0], sc[1][1]), pack_bf16(sc[1][2], sc[1][3])};
#pragma unroll
            for (int j = 0; j < D / 16; ++j) {
                o[2 * j][0] *= alpha_a; o[2 * j][1] *= alpha_a; o[2 * j][2] *= alpha_b; o[2 * j][3] *= alpha_b;
                o[2 * j + 1][0] *= alpha_a; o[2 * j + 1][1] *= alpha_a; o[2 * j + 1][2] *= alpha_b; o[2 * j + 1][3] *= alpha_b;
                const int key = warp * 16 + (mi & 1) * 8 + ri;
                const int chunk_v = j * 2 + (mi >> 1);
                unsigned b[4];
                ldmatrix_x4_trans(b, v_s + (chunk_v >> 3) * kBlockBytes + key * 128 + (((chunk_v & 7) ^ (key & 7)) << 4));
                mma_bf16(o[2 * j], pa, b[0], b[1]);
                mma_bf16(o[2 * j + 1], pa, b[2], b[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + s);           // this warp is done with the stage
        }
    }
    __syncthreads();                // every copy has landed and been read: the stages are free for the merge
    if (warp == 4) return;

    // merge the four warps' partial results through shared memory
    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    float* red_o = reinterpret_cast<float*>(smem);                // [4][16][D]
    float* red_ml = red_o + 4 * 16 * D;                           // [4][16][2]
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int col = nt * 8 + (lane & 3) * 2;
        float* dst_a = red_o + ((size_t)warp * 16 + row_a) * D + col;
        float* dst_b = red_o + ((size_t)warp * 16 + row_b) * D + col;
        dst_a[0] = o[nt][0]; dst_a[1] = o[nt][1];
        dst_b[0] = o[nt][2]; dst_b[1] = o[nt][3];
    }
    if ((lane & 3) == 0) {
        red_ml[(warp * 16 + row_a) * 2] = m_a; red_ml[(warp * 16 + row_a) * 2 + 1] = l_a;
        red_ml[(warp * 16 + row_b) * 2] = m_b; red_ml[(warp * 16 + row_b) * 2 + 1] = l_b;
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    for (int idx = tid; idx < group * D; idx += 128) {
        const int g = idx / D, j = idx - g * D;
        float m_star = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m_star = fmaxf(m_star, red_ml[(w * 16 + g) * 2]);
        float acc = 0.0f, l_sum = 0.0f;
        if (m_star != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float weight = exp2f(red_ml[(w * 16 + g) * 2] - m_star);
                acc += weight * red_o[((size_t)w * 16 + g) * D + j];
                l_sum += weight * red_ml[(w * 16 + g) * 2 + 1];
            }
        }
        const size_t head = (size_t)request * nq + (size_t)kv_head * group + g;
        if (splits == 1) {
            out[head * D + j] = __float2bfloat16_rn(l_sum > 0.0f ? acc / l_sum : 0.0f);
        } else {
            partial_o[(head * splits + split) * D + j] = acc;
            if (j == 0) {
                partial_ml[(head * splits + split) * 2] = m_star;
                partial_ml[(head * splits + split) * 2 + 1] = l_sum;
            }
        }
    }
}

template <int D, bool FUSED>
int launch_decode_tma(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* q, void* out,
                      float* partial_o, float* partial_ml, const int* seq_lens, const int* block_table,
                      int num_requests, int max_pages, int nq, int nkv, int page_size, float scale, int window,
                      int splits, int* error_flag, cudaStream_t stream, DecodeRope rope = DecodeRope()) {
    auto kernel = decode_attention_tma_kernel<D, FUSED>;
    const int smem = kDtStages * 2 * (D / 64) * kKeys * 128 + 64 + 1024 + (FUSED ? decode_rope_smem<D>() : 0);
    static bool configured = false;
    if (!configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (status != cudaSuccess) return fail("decode_attention", cudaGetErrorString(status));
        configured = true;
    }
    dim3 grid(splits, nkv, num_requests);
    launch_overlapped(kernel, grid, kDtThreads, smem, stream, map_k, map_v, (const bf16*)q, (bf16*)out, partial_o,
                      partial_ml, seq_lens, block_table, max_pages, nq, nkv, page_size, scale * kLog2e, window,
                      splits, error_flag, rope);
    if (int rc = check_launch("decode_attention")) return rc;
    if (splits > 1) {
        launch_overlapped(merge_splits_kernel<D>, num_requests * nq, D < 128 ? D : 128, 0, stream,
                          (const float*)partial_o, (const float*)partial_ml, (bf16*)out, splits);
        return check_launch("merge_splits");
    }
    return 0;
}

}  // namespace b200

// bfloat16 paged attention on the tensor cores: one kernel for decode batches
// (one new token per request, keys split over several blocks and merged) and one
// for everything else (portions of prompts, any mix of query lengths).
//
// Both read keys and values page by page through the block table into shared
// memory with 16-byte asynchronous copies (two stages), form scores and outputs
// with m16n8k16 bfloat16 tensor-core products accumulating in float32, and keep
// the softmax statistics (running maximum, running sum) in float32; the
// probabilities are rounded to bfloat16 only as an operand of the second product.
// Masking and the meaning of the arguments are those of attention_generic.cu.
// The split over keys with partial (maximum, sum, output) triples follows the
// scheme of minivllm/attention/ops/triton_unified_attention.py:366-388, 403-478.
//
// Shared-memory tiles are [64 keys][D] with the 16-byte chunks of a row permuted
// by (chunk ^ (row & 7)) so that ldmatrix reads are free of bank conflicts.
#pragma once

#include "common.cuh"

namespace b200 {

using bf16 = __nv_bfloat16;
constexpr int kKeys = 64;          // keys per shared-memory tile
constexpr int kThreads = 128;      // four warps
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Keys k0 .. k0+63 of one request and key/value head into a stage of shared memory.
// Positions at or beyond k_end, and pages that were given back, are filled with zeros.
// A thread always copies the same 16-byte chunk of its rows, so the only per-row work
// is the look-up of the row's page (a shift when the page size is a power of two).
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* k_s, bf16* v_s, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages,
                                             const int* __restrict__ table, int k0, int k_end,
                                             int kv_head, int nkv, int page_size, int page_shift) {
    constexpr int kChunks = D / 8;
    constexpr int kRowsPerPass = kThreads / kChunks;
    const int chunk = threadIdx.x % kChunks, first_row = threadIdx.x / kChunks;
    const size_t in_page = (size_t)kv_head * page_size * D + chunk * 8;
    const size_t page_stride = (size_t)nkv * page_size * D;
#pragma unroll
    for (int i = 0; i < kKeys / kRowsPerPass; ++i) {
        const int row = first_row + i * kRowsPerPass;
        const int kp = k0 + row;
        const int at_s = row * D + ((chunk ^ (row & 7)) << 3);
        int page = -1, offset = 0;
        if (kp < k_end) {
            const int index = page_shift >= 0 ? kp >> page_shift : kp / page_size;
            offset = page_shift >= 0 ? kp & (page_size - 1) : kp - index * page_size;
            page = table[index];
        }
        if (page >= 0) {
            const size_t at = (size_t)page * page_stride + in_page + (size_t)offset * D;
            cp_async16(k_s + at_s, k_pages + at);
            cp_async16(v_s + at_s, v_pages + at);
        } else {
            *reinterpret_cast<uint4*>(k_s + at_s) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(v_s + at_s) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Query rows of a 16-row fragment straight from global memory; rows that do not
// exist are zeros.  row_ptr_a / row_ptr_b: the thread's two rows (lane/4 and +8).
template <int D>
__device__ __forceinline__ void load_q_fragments(unsigned (&qa)[D / 16][4], const bf16* row_a,
                                                 const bf16* row_b, int lane) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int col = ks * 16 + (lane & 3) * 2;
        qa[ks][0] = row_a ? *reinterpret_cast<const unsigned*>(row_a + col) : 0u;
        qa[ks][1] = row_b ? *reinterpret_cast<const unsigned*>(row_b + col) : 0u;
        qa[ks][2] = row_a ? *reinterpret_cast<const unsigned*>(row_a + col + 8) : 0u;
        qa[ks][3] = row_b ? *reinterpret_cast<const unsigned*>(row_b + col + 8) : 0u;
    }
}

// ------------------------------------------------------------------- decode
// grid (splits, kv heads, requests); every request has exactly one query token,
// so token index == request index.  Rows of the 16-row fragment are the query
// heads that share this key/value head (at most 16).
template <int D>
__global__ void __launch_bounds__(kThreads) decode_attention_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    bf16* __restrict__ out, float* __restrict__ partial_o, float* __restrict__ partial_ml,
    const int* __restrict__ seq_lens, const int* __restrict__ block_table, int max_pages, int nq,
    int nkv, int page_size, float scale_log2, int window, int splits) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);
    overlap_trigger();
    overlap_wait();
    const int split = blockIdx.x, kv_head = blockIdx.y, request = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = nq / nkv;
    const int seq_len = seq_lens[request];
    const int k_first = window > 0 ? max(0, seq_len - window) : 0;
    const int total = seq_len - k_first;
    int chunk = (total + splits - 1) / splits;
    chunk = ((chunk + kKeys - 1) / kKeys) * kKeys;
    const int my_begin = k_first + split * chunk;
    const int my_end = min(seq_len, my_begin + chunk);
    const int tiles = my_end > my_begin ? (my_end - my_begin + kKeys - 1) / kKeys : 0;
    const int* table = block_table + (size_t)request * max_pages;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

    const int row_a = lane >> 2, row_b = row_a + 8;
    const bf16* q_base = q + ((size_t)request * nq + (size_t)kv_head * group) * D;
    unsigned qa[D / 16][4];
    load_q_fragments<D>(qa, row_a < group ? q_base + (size_t)row_a * D : nullptr,
                        row_b < group ? q_base + (size_t)row_b * D : nullptr, lane);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;

    auto k_stage = [&](int s) { return stage_base + (size_t)s * 2 * kKeys * D; };
    auto v_stage = [&](int s) { return stage_base + (size_t)s * 2 * kKeys * D + kKeys * D; };

    if (tiles > 0) {
        load_kv_tile<D>(k_stage(0), v_stage(0), k_pages, v_pages, table, my_begin, my_end, kv_head, nkv, page_size, page_shift);
        cp_async_commit();
    }
    for (int t = 0; t < tiles; ++t) {
        const int k0 = my_begin + t * kKeys;
        if (t + 1 < tiles) {
            load_kv_tile<D>(k_stage((t + 1) & 1), v_stage((t + 1) & 1), k_pages, v_pages, table,
                            k0 + kKeys, my_end, kv_head, nkv, page_size, page_shift);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const bf16* k_s = k_stage(t & 1);
        const bf16* v_s = v_stage(t & 1);

        // scores of this warp's 16 keys
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int mi = lane >> 3, ri = lane & 7;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int key = warp * 16 + (mi >> 1) * 8 + ri;
            const int chunk_k = ks * 2 + (mi & 1);
            unsigned b[4];
            ldmatrix_x4(b, k_s + key * D + ((chunk_k ^ (key & 7)) << 3));
            mma_bf16(s[0], qa[ks], b[0], b[1]);
            mma_bf16(s[1], qa[ks], b[2], b[3]);
        }
        float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kp = k0 + warp * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
                const float v = kp < my_end ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
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
            s[nt][0] = exp2f(s[nt][0] - ref_a);
            s[nt][1] = exp2f(s[nt][1] - ref_a);
            s[nt][2] = exp2f(s[nt][2] - ref_b);
            s[nt][3] = exp2f(s[nt][3] - ref_b);
            sum_a += s[nt][0] + s[nt][1];
            sum_b += s[nt][2] + s[nt][3];
        }
        l_a = l_a * alpha_a + sum_a;
        l_b = l_b * alpha_b + sum_b;
        unsigned pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                          pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
            o[2 * j][0] *= alpha_a; o[2 * j][1] *= alpha_a; o[2 * j][2] *= alpha_b; o[2 * j][3] *= alpha_b;
            o[2 * j + 1][0] *= alpha_a; o[2 * j + 1][1] *= alpha_a; o[2 * j + 1][2] *= alpha_b; o[2 * j + 1][3] *= alpha_b;
            const int key = warp * 16 + (mi & 1) * 8 + ri;
            const int chunk_v = j * 2 + (mi >> 1);
            unsigned b[4];
            ldmatrix_x4_trans(b, v_s + key * D + ((chunk_v ^ (key & 7)) << 3));
            mma_bf16(o[2 * j], pa, b[0], b[1]);
            mma_bf16(o[2 * j + 1], pa, b[2], b[3]);
        }
        __syncthreads();
    }

    // merge the four warps' partial results through shared memory
    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    float* red_o = reinterpret_cast<float*>(smem_raw);            // [4][16][D]
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
    __syncthreads();
    for (int idx = tid; idx < group * D; idx += kThreads) {
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

// One block per (token, query head): merge the splits' partial results.  Up to 16 splits
// are fetched in one go (every load issued before any is used); more run through a loop.
template <int D>
__global__ void merge_splits_kernel(const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                                    bf16* __restrict__ out, int splits) {
    overlap_trigger();
    overlap_wait();
    const size_t head = blockIdx.x;
    constexpr int kHeld = 16;
    if (splits <= kHeld) {
        for (int j = threadIdx.x; j < D; j += blockDim.x) {
            float m[kHeld], l[kHeld], o[kHeld];
#pragma unroll
            for (int s = 0; s < kHeld; ++s) {
                const bool in = s < splits;
                m[s] = in ? partial_ml[(head * splits + s) * 2] : -INFINITY;
                l[s] = in ? partial_ml[(head * splits + s) * 2 + 1] : 0.0f;
                o[s] = in ? partial_o[(head * splits + s) * D + j] : 0.0f;
            }
            float m_star = -INFINITY;
#pragma unroll
            for (int s = 0; s < kHeld; ++s) m_star = fmaxf(m_star, m[s]);
            float acc = 0.0f, l_sum = 0.0f;
            if (m_star != -INFINITY) {
#pragma unroll
                for (int s = 0; s < kHeld; ++s) {
                    if (s < splits) {
                        const float weight = exp2f(m[s] - m_star);
                        acc += weight * o[s];
                        l_sum += weight * l[s];
                    }
                }
            }
            out[head * D + j] = __float2bfloat16_rn(l_sum > 0.0f ? acc / l_sum : 0.0f);
        }
        return;
    }
    float m_star = -INFINITY;
    for (int s = 0; s < splits; ++s) m_star = fmaxf(m_star, partial_ml[(head * splits + s) * 2]);
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float acc = 0.0f, l_sum = 0.0f;
        if (m_star != -INFINITY) {
            for (int s = 0; s < splits; ++s) {
                const float weight = exp2f(partial_ml[(head * splits + s) * 2] - m_star);
                acc += weight * partial_o[(head * splits + s) * D + j];
                l_sum += weight * partial_ml[(head * splits + s) * 2 + 1];
            }
        }
        out[head * D + j] = __float2bfloat16_rn(l_sum > 0.0f ? acc / l_sum : 0.0f);
    }
}

// ------------------------------------------------------------------ prefill
// grid (query tiles, query heads).  A tile is 64 consecutive query tokens of one
// request, 16 per warp; the request of a tile is found from the tile index as in
// attention_generic.cu (request r owns tiles [start[r] / 64 + r, start[r+1] / 64 + r + 1)).
template <int D>
__global__ void __launch_bounds__(kThreads, 3) prefill_attention_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
    bf16* __restrict__ out, const int* __restrict__ query_start, const int* __restrict__ seq_lens,
    const int* __restrict__ block_table, int num_requests, int max_pages, int nq, int nkv,
    int page_size, float scale_log2, int window, int token_offset) {
    // token_offset: row of q and out at which the first of these requests begins (requests ahead of
    // them in the batch are another launch's); query_start holds rows of the whole batch.
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* stage_base = reinterpret_cast<bf16*>(smem_raw);
    constexpr int kRows = 64;
    // Late tiles of a long request have the most keys to visit: hand them out first, so
    // that the short ones fill the end of the launch.
    const int block = gridDim.x - 1 - blockIdx.x;
    int lo = 0, hi = num_requests - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((query_start[mid] - token_offset) / kRows + mid <= block) lo = mid; else hi = mid - 1;
    }
    const int request = lo;
    const int q_begin = query_start[request];
    const int q_len = query_start[request + 1] - q_begin;
    const int tile_first = (block - ((q_begin - token_offset) / kRows + request)) * kRows;
    if (tile_first >= q_len) return;
    const int rows_here = min(kRows, q_len - tile_first);
    const int seq_len = seq_lens[request];
    const int past = seq_len - q_len;
    const int head = blockIdx.y;
    const int kv_head = head / (nq / nkv);
    const int* table = block_table + (size_t)request * max_pages;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    const bf16* q_tile = q + ((size_t)(q_begin + tile_first) * nq + head) * D;
    unsigned qa[D / 16][4];
    load_q_fragments<D>(qa, row_a < rows_here ? q_tile + (size_t)row_a * nq * D : nullptr,
                        row_b < rows_here ? q_tile + (size_t)row_b * nq * D : nullptr, lane);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;

    const int first_pos = past + tile_first;
    const int last_pos = first_pos + rows_here - 1;
    const int pos_a = first_pos + row_a, pos_b = first_pos + row_b;
    const int warp_last_pos = first_pos + min(warp * 16 + 15, rows_here - 1);
    const int warp_first_pos = first_pos + warp * 16;
    const int k_first = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int k_end = last_pos + 1;
    const int tiles = (k_end - k_first + kKeys - 1) / kKeys;

    auto k_stage = [&](int s) { return stage_base + (size_t)s * 2 * kKeys * D; };
    auto v_stage = [&](int s) { return stage_base + (size_t)s * 2 * kKeys * D + kKeys * D; };

    load_kv_tile<D>(k_stage(0), v_stage(0), k_pages, v_pages, table, k_first, k_end, kv_head, nkv, page_size, page_shift);
    cp_async_commit();
    for (int t = 0; t < tiles; ++t) {
        const int k0 = k_first + t * kKeys;
        if (t + 1 < tiles) {
            load_kv_tile<D>(k_stage((t + 1) & 1), v_stage((t + 1) & 1), k_pages, v_pages, table,
                            k0 + kKeys, k_end, kv_head, nkv, page_size, page_shift);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // A warp whose rows all lie before this tile (causal) or after its window has nothing to add.
        bool active = warp * 16 < rows_here && k0 <= warp_last_pos;
        if (window > 0 && k0 + kKeys - 1 <= warp_first_pos - window) active = false;
        if (active) {
            const bf16* k_s = k_stage(t & 1);
            const bf16* v_s = v_stage(t & 1);
            const int mi = lane >> 3, ri = lane & 7;
            float s[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    const int key = np * 16 + (mi >> 1) * 8 + ri;
                    const int chunk_k = ks * 2 + (mi & 1);
                    unsigned b[4];
                    ldmatrix_x4(b, k_s + key * D + ((chunk_k ^ (key & 7)) << 3));
                    mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
                }
            }
            float max_a = -INFINITY, max_b = -INFINITY;
            // A tile wholly before the warp's first query (and inside every window) needs no mask.
            const bool all_visible = k0 + kKeys - 1 <= warp_first_pos &&
                                     (window <= 0 || k0 > warp_last_pos - window);
            if (all_visible) {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = s[nt][e] * scale_log2;
                        s[nt][e] = v;
                        if (e < 2) max_a = fmaxf(max_a, v); else max_b = fmaxf(max_b, v);
                    }
            } else {
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int kp = k0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int q_pos = e < 2 ? pos_a : pos_b;
                        bool visible = kp <= q_pos;
                        if (window > 0) visible = visible && (kp > q_pos - window);
                        const float v = visible ? s[nt][e] * scale_log2 : -INFINITY;
                        s[nt][e] = v;
                        if (e < 2) max_a = fmaxf(max_a, v); else max_b = fmaxf(max_b, v);
                    }
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
            for (int nt = 0; nt < 8; ++nt) {
                s[nt][0] = exp2f(s[nt][0] - ref_a);
                s[nt][1] = exp2f(s[nt][1] - ref_a);
                s[nt][2] = exp2f(s[nt][2] - ref_b);
                s[nt][3] = exp2f(s[nt][3] - ref_b);
                sum_a += s[nt][0] + s[nt][1];
                sum_b += s[nt][2] + s[nt][3];
            }
            l_a = l_a * alpha_a + sum_a;
            l_b = l_b * alpha_b + sum_b;
#pragma unroll
            for (int nt = 0; nt < D / 8; ++nt) {
                o[nt][0] *= alpha_a; o[nt][1] *= alpha_a; o[nt][2] *= alpha_b; o[nt][3] *= alpha_b;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const unsigned pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                        pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int j = 0; j < D / 16; ++j) {
                    const int key = kk * 16 + (mi & 1) * 8 + ri;
                    const int chunk_v = j * 2 + (mi >> 1);
                    unsigned b[4];
                    ldmatrix_x4_trans(b, v_s + key * D + ((chunk_v ^ (key & 7)) << 3));
                    mma_bf16(o[2 * j], pa, b[0], b[1]);
                    mma_bf16(o[2 * j + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }

    l_a = quad_sum(l_a);
    l_b = quad_sum(l_b);
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
    bf16* out_tile = out + ((size_t)(q_begin + tile_first) * nq + head) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int col = nt * 8 + (lane & 3) * 2;
        if (row_a < rows_here)
            *reinterpret_cast<unsigned*>(out_tile + (size_t)row_a * nq * D + col) = pack_bf16(o[nt][0] * inv_a, o[nt][1] * inv_a);
        if (row_b < rows_here)
            *reinterpret_cast<unsigned*>(out_tile + (size_t)row_b * nq * D + col) = pack_bf16(o[nt][2] * inv_b, o[nt][3] * inv_b);
    }
}

template <int D>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* partial_o,
                  float* partial_ml, const int* seq_lens, const int* block_table, int num_requests,
                  int max_pages, int nq, int nkv, int page_size, float scale, int window, int splits,
                  cudaStream_t stream) {
    auto kernel = decode_attention_kernel<D>;
    const int smem = 2 * 2 * kKeys * D * (int)sizeof(bf16);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (status != cudaSuccess) return fail("decode_attention", cudaGetErrorString(status));
    dim3 grid(splits, nkv, num_requests);
    launch_overlapped(kernel, grid, kThreads, smem, stream,
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, partial_o, partial_ml,
        seq_lens, block_table, max_pages, nq, nkv, page_size, scale * kLog2e, window, splits);
    if (int rc = check_launch("decode_attention")) return rc;
    if (splits > 1) {
        launch_overlapped(merge_splits_kernel<D>, num_requests * nq, D < 128 ? D : 128, 0, stream,
                          (const float*)partial_o, (const float*)partial_ml, (bf16*)out, splits);
        return check_launch("merge_splits");
    }
    return 0;
}

template <int D>
int launch_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                   const int* query_start, const int* seq_lens, const int* block_table,
                   int num_requests, int num_tokens, int max_pages, int nq, int nkv, int page_size,
                   float scale, int window, int token_offset, cudaStream_t stream) {
    auto kernel = prefill_attention_kernel<D>;
    const int smem = 2 * 2 * kKeys * D * (int)sizeof(bf16);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (status != cudaSuccess) return fail("prefill_attention", cudaGetErrorString(status));
    dim3 grid((num_tokens - token_offset) / 64 + num_requests, nq);
    kernel<<<grid, kThreads, smem, stream>>>(
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, (bf16*)out, query_start, seq_lens,
        block_table, num_requests, max_pages, nq, nkv, page_size, scale * kLog2e, window, token_offset);
    return check_launch("prefill_attention");
}

}  // namespace b200

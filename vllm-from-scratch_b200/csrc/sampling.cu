// Sampling on the device: penalties, the mask of stop tokens, and one kernel that
// turns a row of float32 logits into a token: greedy argmax, or temperature ->
// min-p -> top-k -> top-p -> a draw, as the reference orders them
// (minivllm/sample/sampler.py:243-288, minivllm/sample/ops/topk_topp_sampler.py:48-90).
//
// Instead of sorting the vocabulary, each filter is a threshold on the scaled
// logit found by radix selection over the order-preserving integer image of the
// float (four passes of 256 bins): top-k by counts, top-p by probability mass in
// 2^-40 fixed point, so that the sums do not depend on the order of the atomics
// and a seed always reproduces its tokens.  Ties at a threshold are all kept (the
// reference keeps ties at the k-th value too, and breaks top-p ties by sort order).
// The draw is Gumbel-max: argmax(x_i - log(E_i)), E_i exponential from Philox
// keyed by (seed, index of the generated token, token id), equal in distribution
// to the reference's argmax(p_i / E_i); the keying follows minivllm/worker/gpu/
// sample/gumbel.py:94-131 (the stream depends on the position, not on call order).
#include <curand_kernel.h>

#include "common.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgMax {
    float value;
    int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax mine, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        ArgMax other;
        other.value = __shfl_xor_sync(0xffffffffu, mine.value, offset);
        other.index = __shfl_xor_sync(0xffffffffu, mine.index, offset);
        mine = better(mine, other);
    }
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        ArgMax v = lane < warps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            ArgMax other;
            other.value = __shfl_xor_sync(0xffffffffu, v.value, offset);
            other.index = __shfl_xor_sync(0xffffffffu, v.index, offset);
            v = better(v, other);
        }
        if (lane == 0) scratch[32] = v;
    }
    __syncthreads();
    ArgMax result = scratch[32];
    __syncthreads();
    return result;
}

// One block per row.
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ draw_index,
    int* __restrict__ tokens, float greedy_eps) {
    __shared__ ArgMax arg_scratch[33];
    __shared__ unsigned long long bins[256];
    __shared__ unsigned prefix_key;
    __shared__ unsigned long long carry;

    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * vocab;
    const int tid = threadIdx.x;
    const float temp = temperature[row];

    if (temp < greedy_eps) {
        ArgMax mine{-INFINITY, 0x7fffffff};
        if ((vocab & 3) == 0 && ((uintptr_t)x & 15) == 0) {
            // four 16-byte loads in flight per thread: one block has a whole row to itself
            const float4* x4 = reinterpret_cast<const float4*>(x);
            const int quads = vocab >> 2;
#pragma unroll 4
            for (int i = tid; i < quads; i += blockDim.x) {
                const float4 v = x4[i];
                mine = better(mine, ArgMax{v.x, 4 * i});
                mine = better(mine, ArgMax{v.y, 4 * i + 1});
                mine = better(mine, ArgMax{v.z, 4 * i + 2});
                mine = better(mine, ArgMax{v.w, 4 * i + 3});
            }
        } else {
            for (int i = tid; i < vocab; i += blockDim.x) mine = better(mine, ArgMax{x[i], i});
        }
        mine = block_argmax(mine, arg_scratch);
        if (tid == 0) tokens[row] = mine.index;
        return;
    }

    // Scaled logits y = x / T; maximum and normaliser.
    ArgMax top{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += blockDim.x) top = better(top, ArgMax{x[i] / temp, i});
    top = block_argmax(top, arg_scratch);
    const float y_max = top.value;

    unsigned cut = 0;                       // keep tokens whose key >= cut
    const float mp = min_p[row];
    if (mp > 0.0f) cut = ordered_key(y_max + logf(mp));

    // ---- top-k: the k-th largest key among the kept ones -------------------
    const int k = top_k[row];
    if (k > 0 && k < vocab) {
        unsigned prefix = 0;
        int remaining = k;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int b = tid; b < 256; b += blockDim.x) bins[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab; i += blockDim.x) {
                const unsigned key = ordered_key(x[i] / temp);
                if (key >= cut && (key & mask) == prefix)
                    atomicAdd(&bins[(key >> shift) & 255u], 1ull);
            }
            __syncthreads();
            if (tid == 0) {
                int b = 255;
                unsigned long long above = 0;
                for (; b > 0; --b) {
                    if (above + bins[b] >= (unsigned long long)remaining) break;
                    above += bins[b];
                }
                prefix_key = prefix | ((unsigned)b << shift);
                carry = above;
            }
            __syncthreads();
            prefix = prefix_key;
            remaining -= (int)carry;
            __syncthreads();
        }
        if (prefix > cut) cut = prefix;
    }

    // ---- top-p: drop the smallest tokens while their mass stays <= 1 - p ----
    const float p = top_p[row];
    if (p < 1.0f) {
        const double kFixed = 1099511627776.0;     // 2^40
        unsigned long long local = 0;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const float y = x[i] / temp;
            if (ordered_key(y) >= cut) local += (unsigned long long)((double)expf(y - y_max) * kFixed);
        }
        for (int b = tid; b < 256; b += blockDim.x) bins[b] = 0ull;
        __syncthreads();
        atomicAdd(&bins[0], local);
        __syncthreads();
        const unsigned long long total = bins[0];
        const unsigned long long target = (unsigned long long)((double)total * (double)(1.0f - p));
        unsigned prefix = 0;
        unsigned long long below = 0;              // mass of kept tokens with a smaller key
        __syncthreads();
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int b = tid; b < 256; b += blockDim.x) bins[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab; i += blockDim.x) {
                const float y = x[i] / temp;
                const unsigned key = ordered_key(y);
                if (key >= cut && (key & mask) == prefix)
                    atomicAdd(&bins[(key >> shift) & 255u],
                              (unsigned long long)((double)expf(y - y_max) * kFixed));
            }
            __syncthreads();
            if (tid == 0) {
                int b = 0;
                unsigned long long mass = below;
                for (; b < 255; ++b) {
                    if (mass + bins[b] > target) break;   // this bin holds the first kept token
                    mass += bins[b];
                }
                prefix_key = prefix | ((unsigned)b << shift);
                carry = mass;
            }
            __syncthreads();
            prefix = prefix_key;
            below = carry;
            __syncthreads();
        }
        if (prefix > cut) cut = prefix;
        const unsigned top_key = ordered_key(y_max);
        if (cut > top_key) cut = top_key;          // the largest token always stays
    }

    // ---- the draw ------------------------------------------------------------
    const unsigned long long seed = seeds[row], draw = draw_index[row];
    ArgMax best{-INFINITY, 0x7fffffff};
    const int chunks = (vocab + 3) >> 2;
    for (int c = tid; c < chunks; c += blockDim.x) {
        curandStatePhilox4_32_10_t state;
        curand_init(seed, draw, 4ull * (unsigned long long)c, &state);
        const float4 u = curand_uniform4(&state);
        const float us[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * c + j;
            if (i >= vocab) break;
            const float y = x[i] / temp;
            if (ordered_key(y) < cut) continue;
            const float e = fmaxf(-logf(us[j]), 1e-30f);
            best = better(best, ArgMax{y - logf(e), i});
        }
    }
    best = block_argmax(best, arg_scratch);
    if (tid == 0) tokens[row] = best.index == 0x7fffffff ? top.index : best.index;
}

// Penalties on the distinct tokens a request has seen, listed per row in CSR form:
// tokens[offsets[r] .. offsets[r+1]) with the number of times each occurred in the
// output (0 = prompt only).  minivllm/sample/ops/penalties.py:51-72: a seen token's
// logit is divided by the repetition penalty when positive, multiplied when not;
// then frequency * count and presence * [count > 0] are subtracted.
__global__ void penalties_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ offsets,
                                 const int* __restrict__ seen_tokens, const int* __restrict__ output_counts,
                                 const float* __restrict__ repetition, const float* __restrict__ frequency,
                                 const float* __restrict__ presence) {
    const int row = blockIdx.x;
    float* x = logits + (size_t)row * vocab;
    for (int i = offsets[row] + threadIdx.x; i < offsets[row + 1]; i += blockDim.x) {
        const int token = seen_tokens[i];
        if (token < 0 || token >= vocab) continue;
        float v = x[token];
        const float rep = repetition[row];
        v = v > 0.0f ? v * (1.0f / rep) : v * rep;
        const int count = output_counts[i];
        v -= frequency[row] * (float)count;
        if (count > 0) v -= presence[row];
        x[token] = v;
    }
}

// logits[rows[i], tokens[i]] = -inf: stop tokens of requests that have not yet
// produced their minimum number of tokens (minivllm/sample/sampler.py:73-120).
__global__ void mask_tokens_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                                   const int* __restrict__ tokens, int count) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && tokens[i] >= 0 && tokens[i] < vocab)
        logits[(size_t)rows[i] * vocab + tokens[i]] = -INFINITY;
}

}  // namespace b200

B200_EXPORT int b200_sample(const float* logits, int rows, int vocab, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p,
                            const unsigned long long* seeds, const unsigned long long* draw_index,
                            int* tokens, float greedy_eps, cudaStream_t stream) {
    using namespace b200;
    if (rows == 0) return 0;
    if (vocab <= 0) return fail("sample", "vocabulary must be positive");
    sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, vocab, temperature, top_k, top_p, min_p,
                                                       seeds, draw_index, tokens, greedy_eps);
    return check_launch("sample");
}

B200_EXPORT int b200_penalties(float* logits, int rows, int vocab, const int* offsets,
                               const int* seen_tokens, const int* output_counts, const float* repetition,
                               const float* frequency, const float* presence, cudaStream_t stream) {
    using namespace b200;
    if (rows == 0) return 0;
    penalties_kernel<<<rows, 256, 0, stream>>>(logits, vocab, offsets, seen_tokens, output_counts,
                                               repetition, frequency, presence);
    return check_launch("penalties");
}

B200_EXPORT int b200_mask_tokens(float* logits, int vocab, const int* rows, const int* tokens, int count,
                                 cudaStream_t stream) {
    using namespace b200;
    if (count == 0) return 0;
    mask_tokens_kernel<<<(count + 255) / 256, 256, 0, stream>>>(logits, vocab, rows, tokens, count);
    return check_launch("mask_tokens");
}

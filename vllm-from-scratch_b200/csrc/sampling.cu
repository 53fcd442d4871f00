// Sampling on the device: penalties, the mask of stop tokens, and two kernels (one for rows
// without a filter, one for rows with) that turn a row of float32 logits into a token: greedy argmax, or temperature ->
// min-p -> top-k -> top-p -> a draw, as the reference orders them
// (minivllm/sample/sampler.py:243-288, minivllm/sample/ops/topk_topp_sampler.py:48-90).
//
// Instead of sorting the vocabulary, each filter is a threshold on the scaled
// logit found by radix selection over the order-preserving integer image of the
// float (four passes of 256 bins): top-k by counts, top-p by probability mass in
// 2^-40 fixed point, so that the sums do not depend on the order of the atomics
// and a seed always reproduces its tokens.  The selection does not run over the
// whole row: one pass sorts the kept tokens into coarse bins by their distance
// below the maximum, the bin that holds the threshold is copied into shared memory
// (a few thousand keys at most) and the radix selection runs there; only a
// threshold in the far tail, or a bin too crowded for the list, falls back to
// selecting over the row.  Ties at a threshold are all kept (the
// reference keeps ties at the k-th value too, and breaks top-p ties by sort order).
// The draw is Gumbel-max: argmax(x_i - log(E_i)), E_i exponential from Philox
// keyed by (seed, index of the generated token, token id), equal in distribution
// to the reference's argmax(p_i / E_i); the keying follows minivllm/worker/gpu/
// sample/gumbel.py:94-131 (the stream depends on the position, not on call order).

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
// Calls f(value, index) for every logit of a row, this thread's share.  A block has a whole
// row to itself, so each thread keeps four 16-byte loads in flight where the row allows it.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ x, int vocab, F&& f) {
    const int tid = threadIdx.x, step = blockDim.x;
    if ((vocab & 3) == 0 && ((uintptr_t)x & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int quads = vocab >> 2;
#pragma unroll 4
        for (int i = tid; i < quads; i += step) {
            const float4 v = x4[i];
            f(v.x, 4 * i);
            f(v.y, 4 * i + 1);
            f(v.z, 4 * i + 2);
            f(v.w, 4 * i + 3);
        }
    } else {
        for (int i = tid; i < vocab; i += step) f(x[i], i);
    }
}

__device__ __forceinline__ float key_value(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Probability mass of a scaled logit in 2^-40 fixed point (0 from about 27.7 below the maximum).
// The product with a power of two is exact in float, so this is the floor of exp() * 2^40.
__device__ __forceinline__ unsigned long long fixed_mass(float y, float y_max) {
    return __float2ull_rz(expf(y - y_max) * 1099511627776.0f);
}

// A first, coarse look at a row: kept tokens by how far they lie below the maximum, eight
// bins per unit, the last bin for everything 31.875 and more below.  Bin indices fall as
// the logit rises, so bins are ranges of the key order.  Random-looking logits spread
// over many bins, which keeps the shared-memory atomics apart; the crowded far bin is
// counted in registers.
constexpr int kCoarseBins = 256;
constexpr float kCoarsePerUnit = 8.0f;
constexpr int kListCapacity = 6144;             // candidates of one coarse bin held in shared memory

__device__ __forceinline__ int coarse_bin(float y, float y_max) {
    const float d = (y_max - y) * kCoarsePerUnit;
    return d >= (float)(kCoarseBins - 1) ? kCoarseBins - 1 : (int)d;
}

struct SampleShared {
    ArgMax arg_scratch[33];
    unsigned long long bins[256];               // one radix pass: counts or masses per byte value
    unsigned coarse_mass_lo[kCoarseBins], coarse_mass_hi[kCoarseBins];     // 64-bit sums kept as two words
    unsigned coarse_count[kCoarseBins];
    unsigned list[kListCapacity];               // keys of the kept tokens of one coarse bin
    unsigned list_size;
    unsigned prefix_key;
    unsigned long long carry;
    int chosen_bin;
    unsigned long long chosen_before;           // count above / mass below the chosen bin
};

// The k-th largest key among the keys >= cut that `each` visits (`each(f)` calls f(key) for
// this thread's share).  Fewer than k such keys: the smallest possible prefix, which cuts nothing.
template <typename Each>
__device__ unsigned select_kth_largest(Each&& each, unsigned cut, int k, SampleShared& sh) {
    const int tid = threadIdx.x;
    unsigned prefix = 0;
    int remaining = k;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int b = tid; b < 256; b += blockDim.x) sh.bins[b] = 0ull;
        __syncthreads();
        each([&](unsigned key) {
            if (key >= cut && (key & mask) == prefix) atomicAdd(&sh.bins[(key >> shift) & 255u], 1ull);
        });
        __syncthreads();
        if (tid == 0) {
            int b = 255;
            unsigned long long above = 0;
            for (; b > 0; --b) {
                if (above + sh.bins[b] >= (unsigned long long)remaining) break;
                above += sh.bins[b];
            }
            sh.prefix_key = prefix | ((unsigned)b << shift);
            sh.carry = above;
        }
        __syncthreads();
        prefix = sh.prefix_key;
        remaining -= (int)sh.carry;
        __syncthreads();
    }
    return prefix;
}

// The smallest key at which the mass of the visited keys >= cut, summed from the smallest
// key up and starting from `below`, first exceeds `target`.
template <typename Each>
__device__ unsigned select_mass_from_below(Each&& each, unsigned cut, unsigned long long target,
                                           unsigned long long below, float y_max, SampleShared& sh) {
    const int tid = threadIdx.x;
    unsigned prefix = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int b = tid; b < 256; b += blockDim.x) sh.bins[b] = 0ull;
        __syncthreads();
        each([&](unsigned key) {
            if (key >= cut && (key & mask) == prefix)
                atomicAdd(&sh.bins[(key >> shift) & 255u], fixed_mass(key_value(key), y_max));
        });
        __syncthreads();
        if (tid == 0) {
            int b = 0;
            unsigned long long mass = below;
            for (; b < 255; ++b) {
                if (mass + sh.bins[b] > target) break;       // this bin holds the first kept token
                mass += sh.bins[b];
            }
            sh.prefix_key = prefix | ((unsigned)b << shift);
            sh.carry = mass;
        }
        __syncthreads();
        prefix = sh.prefix_key;
        below = sh.carry;
        __syncthreads();
    }
    return prefix;
}

// Four uniform numbers in (0, 1] for tokens 4 c .. 4 c + 3 of the draw-th generated token of a
// request with this seed: Philox-4x32 with ten rounds (Salmon et al., "Parallel random numbers: as
// easy as 1, 2, 3"), the key the seed, the counter (c, 0, draw).  A function of its arguments
// alone: no state is set up or skipped ahead, which is most of what a generator object costs when
// every group of four tokens has a counter of its own.
__device__ __forceinline__ void philox_uniform4(unsigned long long seed, unsigned long long draw, unsigned c, float (&u)[4]) {
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
    unsigned x0 = c, x1 = 0u, x2 = (unsigned)draw, x3 = (unsigned)(draw >> 32);
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const unsigned hi0 = __umulhi(0xD2511F53u, x0), lo0 = 0xD2511F53u * x0;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, x2), lo1 = 0xCD9E8D57u * x2;
        x0 = hi1 ^ x1 ^ k0;
        x1 = lo1;
        x2 = hi0 ^ x3 ^ k1;
        x3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    const unsigned x[4] = {x0, x1, x2, x3};
#pragma unroll
    for (int j = 0; j < 4; ++j) u[j] = (float)(x[j] >> 8) * 5.9604644775390625e-8f + 2.98023223876953125e-8f;    // (n + 1/2) / 2^24
}

// A row that needs no filter: the argmax, or temperature and a draw with every token kept.
// The host states the same rule when it decides which of the two kernels to launch.
__device__ __forceinline__ bool plain_row(float temp, int k, float p, float mp, float greedy_eps) {
    return temp < greedy_eps || (k <= 0 && p >= 1.0f && mp <= 0.0f);
}

// Plain rows, a cluster of blocks to a row: one pass over the logits (the argmax of x, or of
// x / T - log(E) with the argmax of x / T beside it for a row that holds no finite number), each
// block over every kPlainCluster-th stretch of the row; the blocks' results meet in the shared
// memory of the cluster's first block.  The draw costs a few hundred instructions per four tokens,
// so a row is bound by the instruction rate of the SMs it runs on, not by memory.
constexpr int kPlainCluster = 8;
constexpr int kPlainThreads = 512;

__global__ void __cluster_dims__(kPlainCluster, 1, 1) __launch_bounds__(kPlainThreads) sample_plain_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ draw_index,
    int* __restrict__ tokens, float greedy_eps) {
    __shared__ ArgMax scratch[33];
    __shared__ ArgMax shares[2 * kPlainCluster];        // of the cluster's first block: every block's best and top
    const int row = blockIdx.x / kPlainCluster, tid = threadIdx.x;
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const float temp = temperature[row];
    if (!plain_row(temp, top_k[row], top_p[row], min_p[row], greedy_eps)) return;      // the whole cluster leaves
    const bool greedy = temp < greedy_eps;
    const float* x = logits + (size_t)row * vocab;
    const unsigned long long seed = seeds[row], draw = draw_index[row];
    ArgMax best{-INFINITY, 0x7fffffff}, top{-INFINITY, 0x7fffffff};
    const int chunks = (vocab + 3) >> 2;
    const bool vec = (vocab & 3) == 0 && ((uintptr_t)x & 15) == 0;
    for (int c = (int)rank * kPlainThreads + tid; c < chunks; c += kPlainCluster * kPlainThreads) {
        float xs[4];
        if (vec) {
            const float4 v = reinterpret_cast<const float4*>(x)[c];
            xs[0] = v.x; xs[1] = v.y; xs[2] = v.z; xs[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) xs[j] = 4 * c + j < vocab ? x[4 * c + j] : -INFINITY;
        }
        if (greedy) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (4 * c + j < vocab) best = better(best, ArgMax{xs[j], 4 * c + j});
            continue;
        }
        float us[4];
        philox_uniform4(seed, draw, (unsigned)c, us);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * c + j;
            if (i >= vocab) break;
            const float y = xs[j] / temp;
            top = better(top, ArgMax{y, i});
            const float e = fmaxf(-logf(us[j]), 1e-30f);
            best = better(best, ArgMax{y - logf(e), i});
        }
    }
    best = block_argmax(best, scratch);
    if (!greedy) top = block_argmax(top, scratch);
    if (tid == 0) {
        unsigned mine = (unsigned)__cvta_generic_to_shared(shares + rank), first;
        asm volatile("mapa.shared::cluster.u32 %0, %1, 0;\n" : "=r"(first) : "r"(mine));
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first), "r"(__float_as_uint(best.value)) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 4u), "r"((unsigned)best.index) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 8u * kPlainCluster), "r"(__float_as_uint(top.value)) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 8u * kPlainCluster + 4u), "r"((unsigned)top.index) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    if (rank == 0 && tid < 32) {
        ArgMax b = tid < kPlainCluster ? shares[tid] : ArgMax{-INFINITY, 0x7fffffff};
        ArgMax t = tid < kPlainCluster ? shares[kPlainCluster + tid] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int offset = kPlainCluster / 2; offset > 0; offset >>= 1) {
            b = better(b, ArgMax{__shfl_xor_sync(0xffffffffu, b.value, offset), __shfl_xor_sync(0xffffffffu, b.index, offset)});
            t = better(t, ArgMax{__shfl_xor_sync(0xffffffffu, t.value, offset), __shfl_xor_sync(0xffffffffu, t.index, offset)});
        }
        if (tid == 0) tokens[row] = b.index == 0x7fffffff ? t.index : b.index;
    }
}

// The other rows, one block per row.
__global__ void __launch_bounds__(kSampleThreads, 1) sample_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ draw_index,
    int* __restrict__ tokens, float greedy_eps) {
    __shared__ SampleShared sh;

    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * vocab;
    const int tid = threadIdx.x;
    const float temp = temperature[row];

    if (plain_row(temp, top_k[row], top_p[row], min_p[row], greedy_eps)) return;       // the other kernel's

    // Scaled logits y = x / T; maximum and normaliser.
    ArgMax top{-INFINITY, 0x7fffffff};
    for_each_logit(x, vocab, [&](float v, int i) { top = better(top, ArgMax{v / temp, i}); });
    top = block_argmax(top, sh.arg_scratch);
    const float y_max = top.value;

    unsigned cut = 0;                       // keep tokens whose key >= cut
    const float mp = min_p[row];
    if (mp > 0.0f) cut = ordered_key(y_max + logf(mp));

    auto each_in_row = [&](auto&& f) { for_each_logit(x, vocab, [&](float v, int) { f(ordered_key(v / temp)); }); };
    auto each_in_list = [&](auto&& f) {
        const int n = (int)sh.list_size;
        for (int i = tid; i < n; i += blockDim.x) f(sh.list[i]);
    };
    // Counts (and, for top-p, masses) of the kept tokens per coarse bin.
    // (A mass is added as two 32-bit words with the carry passed on by hand: nearly all
    // masses fit the low word, and 32-bit shared-memory atomics are the fast ones.)
    auto add_mass = [&](int b, unsigned long long m) {
        const unsigned lo = (unsigned)m, hi = (unsigned)(m >> 32);
        const unsigned before = atomicAdd(&sh.coarse_mass_lo[b], lo);
        const unsigned carry = before + lo < before ? 1u : 0u;
        if (hi + carry) atomicAdd(&sh.coarse_mass_hi[b], hi + carry);
    };
    auto mass_of_bin = [&](int b) { return ((unsigned long long)sh.coarse_mass_hi[b] << 32) + sh.coarse_mass_lo[b]; };
    auto look = [&](bool with_mass) {
        for (int b = tid; b < kCoarseBins; b += blockDim.x) sh.coarse_count[b] = sh.coarse_mass_lo[b] = sh.coarse_mass_hi[b] = 0u;
        __syncthreads();
        unsigned far_count = 0;
        unsigned long long far_mass = 0;
        each_in_row([&](unsigned key) {
            if (key < cut) return;
            const float y = key_value(key);
            const int b = coarse_bin(y, y_max);
            if (b == kCoarseBins - 1) {
                ++far_count;
                if (with_mass) far_mass += fixed_mass(y, y_max);
            } else {
                atomicAdd(&sh.coarse_count[b], 1u);
                if (with_mass) add_mass(b, fixed_mass(y, y_max));
            }
        });
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            far_count += __shfl_xor_sync(0xffffffffu, far_count, offset);
            far_mass += __shfl_xor_sync(0xffffffffu, far_mass, offset);
        }
        if ((tid & 31) == 0 && far_count) {
            atomicAdd(&sh.coarse_count[kCoarseBins - 1], far_count);
            add_mass(kCoarseBins - 1, far_mass);
        }
        __syncthreads();
    };
    // The kept tokens of coarse bin `bin` into the list (a warp appends together).
    auto gather = [&](int bin) {
        if (tid == 0) sh.list_size = 0u;
        __syncthreads();
        each_in_row([&](unsigned key) {
            const bool mine = key >= cut && coarse_bin(key_value(key), y_max) == bin;
            const unsigned active = __activemask();
            const unsigned who = __ballot_sync(active, mine);
            if (who == 0u) return;
            const int lane = tid & 31, leader = __ffs(who) - 1;
            unsigned base = 0;
            if (lane == leader) base = atomicAdd(&sh.list_size, (unsigned)__popc(who));
            base = __shfl_sync(active, base, leader);
            if (mine) {
                const unsigned at = base + __popc(who & ((1u << lane) - 1u));
                if (at < (unsigned)kListCapacity) sh.list[at] = key;
            }
        });
        __syncthreads();
    };

    // ---- top-k: the k-th largest key among the kept ones -------------------
    const int k = top_k[row];
    const float p = top_p[row];
    bool looked = false;                    // the coarse bins hold counts and masses under the current cut
    if (k > 0 && k < vocab) {
        look(p < 1.0f);
        looked = true;
        if (tid == 0) {
            unsigned long long above = 0;
            int b = 0;
            for (; b < kCoarseBins; ++b) {
                if (above + sh.coarse_count[b] >= (unsigned long long)k) break;
                above += sh.coarse_count[b];
            }
            sh.chosen_bin = b;                  // kCoarseBins: fewer than k tokens are kept
            sh.chosen_before = above;
        }
        __syncthreads();
        const int bin = sh.chosen_bin;
        const unsigned long long above = sh.chosen_before;
        __syncthreads();
        if (bin < kCoarseBins) {
            unsigned kth;
            if (bin < kCoarseBins - 1 && sh.coarse_count[bin] <= (unsigned)kListCapacity) {
                gather(bin);
                kth = select_kth_largest(each_in_list, cut, k - (int)above, sh);
            } else {
                kth = select_kth_largest(each_in_row, cut, k, sh);         // the far bin, or a crowd: the whole row
            }
            if (kth > cut) { cut = kth; looked = false; }
        }
    }

    // ---- top-p: drop the smallest tokens while their mass stays <= 1 - p ----
    if (p < 1.0f) {
        if (!looked) look(true);
        if (tid == 0) {
            unsigned long long total = 0;
            for (int b = 0; b < kCoarseBins; ++b) total += mass_of_bin(b);
            const unsigned long long target = (unsigned long long)((double)total * (double)(1.0f - p));
            unsigned long long below = 0;
            int b = kCoarseBins - 1;
            for (; b > 0; --b) {
                if (below + mass_of_bin(b) > target) break;
                below += mass_of_bin(b);
            }
            sh.chosen_bin = b;
            sh.chosen_before = below;
            sh.carry = target;
        }
        __syncthreads();
        const int bin = sh.chosen_bin;
        const unsigned long long below = sh.chosen_before, target = sh.carry;
        __syncthreads();
        unsigned edge;
        if (bin < kCoarseBins - 1 && sh.coarse_count[bin] <= (unsigned)kListCapacity) {
            gather(bin);
            edge = select_mass_from_below(each_in_list, cut, target, below, y_max, sh);
        } else {
            edge = select_mass_from_below(each_in_row, cut, target, 0ull, y_max, sh);
        }
        if (edge > cut) cut = edge;
        const unsigned top_key = ordered_key(y_max);
        if (cut > top_key) cut = top_key;          // the largest token always stays
    }

    // ---- the draw ------------------------------------------------------------
    const unsigned long long seed = seeds[row], draw = draw_index[row];
    ArgMax best{-INFINITY, 0x7fffffff};
    const int chunks = (vocab + 3) >> 2;
    const bool vec = (vocab & 3) == 0 && ((uintptr_t)x & 15) == 0;
    for (int c = tid; c < chunks; c += blockDim.x) {
        float xs[4];
        if (vec) {
            const float4 v = reinterpret_cast<const float4*>(x)[c];
            xs[0] = v.x; xs[1] = v.y; xs[2] = v.z; xs[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) xs[j] = 4 * c + j < vocab ? x[4 * c + j] : -INFINITY;
        }
        bool any = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) any = any || (4 * c + j < vocab && ordered_key(xs[j] / temp) >= cut);
        if (!any) continue;                        // no kept token here: its random numbers are not needed
        float us[4];
        philox_uniform4(seed, draw, (unsigned)c, us);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * c + j;
            if (i >= vocab) break;
            const float y = xs[j] / temp;
            if (ordered_key(y) < cut) continue;
            const float e = fmaxf(-logf(us[j]), 1e-30f);
            best = better(best, ArgMax{y - logf(e), i});
        }
    }
    best = block_argmax(best, sh.arg_scratch);
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
                            int* tokens, float greedy_eps, int kinds, cudaStream_t stream) {
    // kinds: bit 0 = some row may be plain (greedy, or temperature alone), bit 1 = some row may
    // have a filter; a kernel none of whose rows can be there is not launched.
    using namespace b200;
    if (rows == 0) return 0;
    if (vocab <= 0) return fail("sample", "vocabulary must be positive");
    if ((kinds & 3) == 0) return fail("sample", "neither kind of row is said to be there");
    if (kinds & 1) {
        sample_plain_kernel<<<rows * kPlainCluster, kPlainThreads, 0, stream>>>(logits, vocab, temperature, top_k, top_p, min_p,
                                                                                seeds, draw_index, tokens, greedy_eps);
        const int status = check_launch("sample (plain rows)");
        if (status) return status;
    }
    if (kinds & 2)
        sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, vocab, temperature, top_k, top_p, min_p,
                                                           seeds, draw_index, tokens, greedy_eps);
    return check_launch("sample");
}

namespace b200 {
__global__ void collect_status_kernel(const int* a, const int* b, const int* c, int* out) {
    if (threadIdx.x == 0) out[0] = a != nullptr ? *a : 0;
    if (threadIdx.x == 1) out[1] = b != nullptr ? *b : 0;
    if (threadIdx.x == 2) out[2] = c != nullptr ? *c : 0;
}
}  // namespace b200

// out[0..2] = the words at a, b, c (0 for a null pointer): the error words that kernels of a step
// may have set, put beside the step's sampled ids so that one copy brings both to the host.
B200_EXPORT int b200_collect_status(const int* a, const int* b, const int* c, int* out, cudaStream_t stream) {
    using namespace b200;
    collect_status_kernel<<<1, 32, 0, stream>>>(a, b, c, out);
    return check_launch("collect_status");
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

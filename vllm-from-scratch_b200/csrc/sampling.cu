// Sampling on the device: penalties, the mask of stop tokens, and two kernels (one for rows
// without a filter, one for rows with) that turn a row of float32 logits into a token: greedy argmax, or temperature ->
// min-p -> top-k -> top-p -> a draw, as the reference orders them
// (minivllm/sample/sampler.py:243-288, minivllm/sample/ops/topk_topp_sampler.py:48-90).
//
// Instead of sorting the vocabulary, each filter is a threshold on the scaled
// logit found by selection: top-k by counts, top-p by probability mass in
// 2^-40 fixed point, so that the sums do not depend on the order of the atomics
// and a seed always reproduces its tokens.  A row is shared by a cluster of eight
// blocks.  One pass sorts the kept tokens into coarse bins by their distance
// below the maximum; the bin that holds the threshold is divided again while it
// holds more tokens than fit into shared memory, then its keys are copied there and
// a radix selection over the order-preserving integer image of the float (four
// passes of 256 bins) runs on them.  Only a threshold in the far tail, or thousands
// of tokens within a few units in the last place of each other, fall back to radix
// selection over the row.  Ties at a threshold are all kept (the
// reference keeps ties at the k-th value too, and breaks top-p ties by sort order).
// The draw is Gumbel-max: argmax(x_i - log(E_i)), E_i exponential from Philox
// keyed by (seed, index of the generated token, token id), equal in distribution
// to the reference's argmax(p_i / E_i); the keying follows minivllm/worker/gpu/
// sample/gumbel.py:94-131 (the stream depends on the position, not on call order).

#include "common.cuh"

namespace b200 {

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

__device__ __forceinline__ float key_value(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Probability mass of a scaled logit in 2^-40 fixed point (0 from about 27.7 below the maximum).
// The product with a power of two is exact in float, so this is the floor of exp() * 2^40.
__device__ __forceinline__ unsigned long long fixed_mass(float y, float y_max) {
    return __float2ull_rz(expf(y - y_max) * 1099511627776.0f);
}

// ---- a cluster of blocks to a row ------------------------------------------------------------
// The blocks of a cluster share a row: each walks over every n-th stretch of it (n blocks), adds
// what it finds to tables in its own shared memory, and after a barrier of the cluster every block
// sums the tables of all (through distributed shared memory) and takes the same decision from the
// same numbers, so that all blocks follow one path and meet at the same barriers.
constexpr int kRowCluster = 8;             // blocks to a row at most (the portable size of a cluster)

__device__ __forceinline__ unsigned cluster_blocks() {
    unsigned n;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(n));
    return n;
}

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

__device__ __forceinline__ unsigned peer_address(const void* mine, unsigned rank) {
    unsigned there;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(there) : "r"((unsigned)__cvta_generic_to_shared(mine)), "r"(rank));
    return there;
}

__device__ __forceinline__ unsigned peer_u32(const void* mine, unsigned rank) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(peer_address(mine, rank)) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long peer_u64(const void* mine, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(v) : "r"(peer_address(mine, rank)) : "memory");
    return v;
}

// The best of the blocks' results: every block has written its own into `mine` (the same place
// in each block's shared memory) before a barrier of the cluster; the first 32 threads call this.
__device__ __forceinline__ ArgMax cluster_best(const ArgMax* mine, unsigned blocks) {
    const int lane = threadIdx.x & 31;
    ArgMax v{-INFINITY, 0x7fffffff};
    if (lane < (int)blocks) {
        v.value = __uint_as_float(peer_u32(&mine->value, (unsigned)lane));
        v.index = (int)peer_u32(&mine->index, (unsigned)lane);
    }
#pragma unroll
    for (int offset = kRowCluster / 2; offset > 0; offset >>= 1)
        v = better(v, ArgMax{__shfl_xor_sync(0xffffffffu, v.value, offset), __shfl_xor_sync(0xffffffffu, v.index, offset)});
    return v;
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
constexpr int kPlainCluster = kRowCluster;
constexpr int kPlainThreads = 512;

__global__ void __cluster_dims__(kPlainCluster, 1, 1) __launch_bounds__(kPlainThreads) sample_plain_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ draw_index,
    int* __restrict__ tokens, float greedy_eps) {
    __shared__ ArgMax scratch[33];
    __shared__ ArgMax shares[2 * kPlainCluster];        // of the cluster's first block: every block's best and top
    const int row = blockIdx.x / kPlainCluster, tid = threadIdx.x;
    const unsigned rank = cluster_rank();
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
        const unsigned first = peer_address(shares + rank, 0u);        // the same place in the first block
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first), "r"(__float_as_uint(best.value)) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 4u), "r"((unsigned)best.index) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 8u * kPlainCluster), "r"(__float_as_uint(top.value)) : "memory");
        asm volatile("st.shared::cluster.b32 [%0], %1;\n" ::"r"(first + 8u * kPlainCluster + 4u), "r"((unsigned)top.index) : "memory");
    }
    cluster_sync();
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

// ---- log-probabilities of what was sampled ---------------------------------------------------
// For a row that wants them: log_softmax of its logits (as they were before penalties, masks and
// temperature: minivllm/sample/sampler.py:86-95, 313-315) at the sampled token, that token's place
// among all tokens (how many logits are at least as large: minivllm/sample/sampler.py:318-349),
// and the `wanted[row]` largest tokens in order (ties by token id).  A cluster of eight blocks to
// a row: one pass for the maximum, the sum of exponentials (pairs of a maximum and a sum, joined
// in a fixed order: the same row gives the same bits in any batch) and the place, then one pass
// for every token of the list, each the largest that comes after the one before it.
//   ids, values: [rows][width], column 0 the sampled token, columns 1 .. wanted[row] the list;
//   place: [rows].  Rows with wanted[row] < 0 are left alone.
constexpr int kLogprobThreads = 512;
constexpr int kMaxLogprobs = 32;

struct SoftmaxPart {
    float top, sum;             // sum of exp(x - top) over a part of the row
};

__device__ __forceinline__ SoftmaxPart join(SoftmaxPart a, SoftmaxPart b) {
    if (b.top == -INFINITY) return a;
    if (a.top == -INFINITY) return b;
    const float top = fmaxf(a.top, b.top);
    return SoftmaxPart{top, a.sum * expf(a.top - top) + b.sum * expf(b.top - top)};
}

__global__ void __cluster_dims__(kRowCluster, 1, 1) __launch_bounds__(kLogprobThreads) logprobs_kernel(
    const float* __restrict__ logits, int vocab, const int* __restrict__ tokens, const int* __restrict__ wanted, int width,
    int* __restrict__ ids, float* __restrict__ values, int* __restrict__ place) {
    __shared__ ArgMax scratch[33];
    __shared__ SoftmaxPart parts[kLogprobThreads / 32];
    __shared__ unsigned counts[kLogprobThreads / 32];
    struct Shown {              // what this block shows to the others, used in turn
        SoftmaxPart part;
        unsigned count;
        ArgMax best;
    };
    __shared__ Shown shown[2];
    __shared__ ArgMax agreed;
    const int row = blockIdx.x / kRowCluster, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned rank = cluster_rank();
    const int n = wanted[row];
    if (n < 0) return;                                  // the whole cluster leaves
    const float* x = logits + (size_t)row * vocab;
    const int token = tokens[row];
    const float x_token = token >= 0 && token < vocab ? x[token] : -INFINITY;
    const int chunks = (vocab + 3) >> 2;
    const bool vec = (vocab & 3) == 0 && ((uintptr_t)x & 15) == 0;
    auto each = [&](auto&& f) {                         // f(logit, token id) over this thread's share of the row
        for (int c = (int)rank * kLogprobThreads + tid; c < chunks; c += kRowCluster * kLogprobThreads) {
            if (vec) {
                const float4 v = reinterpret_cast<const float4*>(x)[c];
                f(v.x, 4 * c); f(v.y, 4 * c + 1); f(v.z, 4 * c + 2); f(v.w, 4 * c + 3);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (4 * c + j < vocab) f(x[4 * c + j], 4 * c + j);
            }
        }
    };
    int turn = 0;

    // maximum, sum of exponentials, place of the sampled token
    SoftmaxPart mine{-INFINITY, 0.0f};
    unsigned at_least = 0;
    each([&](float v, int) {
        if (v > mine.top) {
            mine.sum = mine.sum * expf(mine.top - v) + 1.0f;    // exp(-inf) = 0 for the first
            mine.top = v;
        } else if (v > -INFINITY) {
            mine.sum += expf(v - mine.top);
        }
        at_least += v >= x_token ? 1u : 0u;
    });
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        mine = join(mine, SoftmaxPart{__shfl_xor_sync(0xffffffffu, mine.top, offset), __shfl_xor_sync(0xffffffffu, mine.sum, offset)});
        at_least += __shfl_xor_sync(0xffffffffu, at_least, offset);
    }
    if (lane == 0) {
        parts[warp] = mine;
        counts[warp] = at_least;
    }
    __syncthreads();
    if (tid == 0) {
        SoftmaxPart all = parts[0];
        unsigned count = counts[0];
        for (int w = 1; w < kLogprobThreads / 32; ++w) {
            all = join(all, parts[w]);
            count += counts[w];
        }
        shown[turn].part = all;
        shown[turn].count = count;
    }
    cluster_sync();
    SoftmaxPart whole{-INFINITY, 0.0f};
    unsigned count = 0;
    for (unsigned r = 0; r < (unsigned)kRowCluster; ++r) {          // every thread, the same order
        whole = join(whole, SoftmaxPart{__uint_as_float(peer_u32(&shown[turn].part.top, r)),
                                        __uint_as_float(peer_u32(&shown[turn].part.sum, r))});
        count += peer_u32(&shown[turn].count, r);
    }
    turn ^= 1;
    const float log_sum = whole.top + logf(whole.sum);
    if (rank == 0 && tid == 0) {
        ids[(size_t)row * width] = token;
        values[(size_t)row * width] = x_token - log_sum;
        place[row] = (int)count;
    }

    // the list: each time the largest token that comes after the last one (value falling, id rising)
    ArgMax last{INFINITY, -1};
    for (int j = 0; j < n && j + 1 < width; ++j) {
        ArgMax best{-INFINITY, 0x7fffffff};
        each([&](float v, int i) {
            const bool after = v < last.value || (v == last.value && i > last.index);
            if (after) best = better(best, ArgMax{v, i});
        });
        best = block_argmax(best, scratch);
        if (tid == 0) shown[turn].best = best;
        cluster_sync();
        if (tid < 32) {
            const ArgMax all = cluster_best(&shown[turn].best, (unsigned)kRowCluster);
            if (tid == 0) agreed = all;
        }
        __syncthreads();
        last = agreed;
        turn ^= 1;
        if (rank == 0 && tid == 0) {
            ids[(size_t)row * width + 1 + j] = last.index == 0x7fffffff ? -1 : last.index;
            values[(size_t)row * width + 1 + j] = last.value - log_sum;
        }
        __syncthreads();                                // `agreed` is written again in the next round
    }
    cluster_sync();                                     // no block leaves while another may read what it shows
}

// ---- rows with a filter ------------------------------------------------------------------------
constexpr int kFilterThreads = 1024;         // four threads to each of 256 bins when columns are summed
constexpr int kCoarseBins = 256;
constexpr float kCoarsePerUnit = 8.0f;
constexpr int kListCapacity = 6144;             // candidates of one bin held in a block's shared memory
constexpr int kLevels = 3;                      // a crowded bin is divided again, this often at most

struct Tables {                                 // what a block found in its share of the row
    unsigned long long mass[256];
    unsigned count[256];
    ArgMax arg;
};

// While a block walks over its share of the row, each lane of a warp adds to a column of its own:
// tokens crowd into a few bins, and 32 lanes adding to one word would queue up; 32 columns are 32
// banks, so the lanes of a warp never meet.  A mass (below 2^41) is added as its low 20 bits and
// the rest (2^20 at most): a column takes fewer than 2^12 tokens of a row (the launcher sees to
// that with the number of blocks it gives a row), so neither sum leaves 32 bits.
struct Columns {
    unsigned count[256][32];
    unsigned low[256][32];
    unsigned high[256][32];
};
constexpr int kMassLowBits = 20;
constexpr int kColumnMaxTokens = (1 << (32 - kMassLowBits)) - 1;       // tokens that a lane may add to a column

struct FilterShared {
    Columns columns;
    ArgMax arg_scratch[33];
    Tables mine[2];                             // used in turn: the others may still read the last one
    unsigned long long mass[256];               // the cluster's sums
    unsigned count[256];
    unsigned list[kListCapacity];               // this block's share of the keys of one bin
    unsigned all[kListCapacity];                // those of all blocks
    unsigned list_size, all_size;
    int chosen;
    unsigned long long before;
    ArgMax best;
};

// A 64-bit sum in shared memory as two 32-bit atomics with the carry passed on by hand (32-bit
// shared-memory atomics are the fast ones, and nearly all masses fit the low word).
__device__ __forceinline__ void add_wide(unsigned long long* slot, unsigned long long m) {
    unsigned* words = reinterpret_cast<unsigned*>(slot);
    const unsigned lo = (unsigned)m, hi = (unsigned)(m >> 32);
    const unsigned before = atomicAdd(words, lo);
    const unsigned carry = before + lo < before ? 1u : 0u;
    if (hi + carry) atomicAdd(words + 1, hi + carry);
}

template <bool WITH_MASS>
__device__ __forceinline__ void column_add(Columns& columns, bool in, int bin, unsigned long long m) {
    if (!in) return;
    const int lane = threadIdx.x & 31;
    atomicAdd(&columns.count[bin][lane], 1u);
    if (WITH_MASS) {
        atomicAdd(&columns.low[bin][lane], (unsigned)m & ((1u << kMassLowBits) - 1u));
        const unsigned high = (unsigned)(m >> kMassLowBits);
        if (high) atomicAdd(&columns.high[bin][lane], high);
    }
}

// The first j of 0..255 at which v(0) + .. + v(j) reaches `need` (STRICT: exceeds it), with the sum
// before it; j = 256 and the whole sum if none does.  The first warp works, every thread gets the result.
template <bool STRICT, typename Get>
__device__ void first_crossing(Get&& v, unsigned long long need, FilterShared& sh, int& j_out, unsigned long long& before_out) {
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        unsigned long long mine[8], sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            mine[i] = v(8 * lane + i);
            sum += mine[i];
        }
        unsigned long long upto = sum;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const unsigned long long other = __shfl_up_sync(0xffffffffu, upto, offset);
            if (lane >= offset) upto += other;
        }
        const unsigned who = __ballot_sync(0xffffffffu, STRICT ? upto > need : upto >= need);
        if (who == 0u) {
            if (lane == 31) {
                sh.chosen = 256;
                sh.before = upto;
            }
        } else if (lane == __ffs(who) - 1) {
            unsigned long long run = upto - sum;
            int at = -1;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (at < 0) {
                    if (STRICT ? run + mine[i] > need : run + mine[i] >= need) at = i;
                    else run += mine[i];
                }
            }
            sh.chosen = 8 * lane + at;
            sh.before = run;
        }
    }
    __syncthreads();
    j_out = sh.chosen;
    before_out = sh.before;
    __syncthreads();
}

// Launched with clusters of 2, 4 or 8 blocks (a launch attribute): many rows get fewer blocks each, so
// that all rows run at once.
__global__ void __launch_bounds__(kFilterThreads, 1) sample_filtered_kernel(
    const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
    const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ draw_index,
    int* __restrict__ tokens, float greedy_eps) {
    extern __shared__ __align__(16) unsigned char filter_shared_raw[];
    FilterShared& sh = *reinterpret_cast<FilterShared*>(filter_shared_raw);

    const unsigned rank = cluster_rank(), blocks = cluster_blocks();
    const int row = blockIdx.x / blocks;
    const float* x = logits + (size_t)row * vocab;
    const int tid = threadIdx.x, lane = tid & 31;
    const int stride = (int)blocks * kFilterThreads;        // chunks of four tokens from one of this thread's to its next
    const float temp = temperature[row];
    const int k = top_k[row];
    const float p = top_p[row], mp = min_p[row];
    if (plain_row(temp, k, p, mp, greedy_eps)) return;             // the other kernel's; the whole cluster leaves

    const int chunks = (vocab + 3) >> 2;
    const bool vec = (vocab & 3) == 0 && ((uintptr_t)x & 15) == 0;
    // f(key of the scaled logit x / T, whether there is such a token) for this block's share of
    // the row; the lanes of a warp call f together.
    auto load_chunk = [&](int c, float (&xs)[4]) {      // tokens 4 c .. 4 c + 3, zeros past the row's end
        if (vec) {
            const float4 v = reinterpret_cast<const float4*>(x)[c];
            xs[0] = v.x; xs[1] = v.y; xs[2] = v.z; xs[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) xs[j] = 4 * c + j < vocab ? x[4 * c + j] : 0.0f;
        }
    };
    auto each_in_row = [&](auto&& f) {
        for (int c0 = (int)rank * kFilterThreads + (tid & ~31); c0 < chunks; c0 += stride) {
            const int c = c0 + lane;
            float xs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (c < chunks) load_chunk(c, xs);
#pragma unroll
            for (int j = 0; j < 4; ++j) f(ordered_key(xs[j] / temp), c < chunks && 4 * c + j < vocab);
        }
    };
    auto each_in_all = [&](auto&& f) {              // the keys that the blocks have gathered, the same in every block
        const int n = (int)sh.all_size;
        for (int i = tid; i < n; i += kFilterThreads) f(sh.all[i], true);
    };

    int turn = 0;                           // which of the two tables the next exchange uses
    auto clear_columns = [&](bool with_mass) {
        unsigned* words = &sh.columns.count[0][0];
        const int n = (with_mass ? 3 : 1) * 256 * 32;               // count, low and high lie one behind the other
        for (int i = tid; i < n; i += kFilterThreads) words[i] = 0u;
        __syncthreads();
    };
    // The columns of a bin summed into this block's table: four threads to a bin, eight columns
    // each, taken in an order that keeps the threads of a warp on different banks.
    auto fold_columns = [&](bool with_mass) {
        __syncthreads();
        Tables& t = sh.mine[turn];
        const int b = tid >> 2, q = tid & 3;
        unsigned n = 0;
        unsigned long long low = 0, high = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int column = (8 * q + i + b) & 31;
            n += sh.columns.count[b][column];
            if (with_mass) {
                low += sh.columns.low[b][column];
                high += sh.columns.high[b][column];
            }
        }
        unsigned long long m = low + (high << kMassLowBits);
#pragma unroll
        for (int offset = 1; offset < 4; offset <<= 1) {
            n += __shfl_xor_sync(0xffffffffu, n, offset);
            m += __shfl_xor_sync(0xffffffffu, m, offset);
        }
        if (q == 0) {
            t.count[b] = n;
            t.mass[b] = m;
        }
    };
    auto clear_sums = [&]() {
        for (int b = tid; b < 256; b += kFilterThreads) {
            sh.mass[b] = 0ull;
            sh.count[b] = 0u;
        }
        __syncthreads();
    };
    // After the blocks have filled their tables: the sums over the cluster into sh.mass and
    // sh.count.  A block writes into a table again two exchanges later, when every block has
    // passed the barrier in between and so has read it.
    auto sum_over_cluster = [&]() {
        cluster_sync();
        const Tables& t = sh.mine[turn];
        for (int b = tid; b < 256; b += kFilterThreads) {
            unsigned long long m = 0;
            unsigned n = 0;
            for (unsigned r = 0; r < blocks; ++r) {
                m += peer_u64(&t.mass[b], r);
                n += peer_u32(&t.count[b], r);
            }
            sh.mass[b] = m;
            sh.count[b] = n;
        }
        __syncthreads();
        turn ^= 1;
    };
    auto best_of_cluster = [&](ArgMax mine) {
        mine = block_argmax(mine, sh.arg_scratch);
        if (tid == 0) sh.mine[turn].arg = mine;
        cluster_sync();
        if (tid < 32) {
            const ArgMax all = cluster_best(&sh.mine[turn].arg, blocks);
            if (tid == 0) sh.best = all;
        }
        __syncthreads();
        turn ^= 1;
        return sh.best;
    };

    // Scaled logits y = x / T: the maximum.
    ArgMax top{-INFINITY, 0x7fffffff};
    for (int c = (int)rank * kFilterThreads + tid; c < chunks; c += stride) {
        float xs[4];
        load_chunk(c, xs);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (4 * c + j < vocab) top = better(top, ArgMax{xs[j] / temp, 4 * c + j});
    }
    top = best_of_cluster(top);
    const float y_max = top.value;

    unsigned cut = 0;                       // keep tokens whose key >= cut
    if (mp > 0.0f) cut = ordered_key(y_max + logf(mp));

    // A first, coarse look at the row sorts the kept tokens by how far they lie below the maximum:
    // eight bins per unit, the last bin for everything 31.875 and more below.  Bin numbers fall as
    // the logit rises, so bins are ranges of the key order.  A bin with more tokens than the list
    // holds is divided again into 256 (level 2, and those once more, level 3): `in1`, `in2` name
    // the bins of levels 1 and 2 that are looked into.  The differences are exact, so that a
    // token falls into the same bins at every look.
    auto locate = [&](float y, int level, int in1, int in2, int& bin) -> bool {
        const float d = (y_max - y) * kCoarsePerUnit;
        const int b1 = d >= (float)(kCoarseBins - 1) ? kCoarseBins - 1 : (int)d;
        if (level == 1) {
            bin = b1;
            return true;
        }
        if (b1 != in1) return false;
        const float f2 = (d - (float)in1) * 256.0f;
        const int b2 = min(max((int)f2, 0), 255);
        if (level == 2) {
            bin = b2;
            return true;
        }
        if (b2 != in2) return false;
        bin = min(max((int)((f2 - (float)in2) * 256.0f), 0), 255);
        return true;
    };
    auto look = [&](int level, int in1, int in2, bool with_mass) {
        clear_columns(with_mass);
        each_in_row([&](unsigned key, bool there) {
            const float y = key_value(key);
            int bin = 0;
            const bool in = there && key >= cut && locate(y, level, in1, in2, bin);
            if (with_mass) column_add<true>(sh.columns, in, bin, in ? fixed_mass(y, y_max) : 0ull);
            else column_add<false>(sh.columns, in, bin, 0ull);
        });
        fold_columns(with_mass);
        sum_over_cluster();
    };
    // The kept tokens of bin `bin`: this block's into its list (a warp appends together), then the
    // lists of all blocks into `all`.  A block's list is written again after a later look at the row,
    // whose barrier every block reaches after it has copied.
    auto gather = [&](int level, int in1, int in2, int bin) {
        if (tid == 0) sh.list_size = 0u;
        __syncthreads();
        each_in_row([&](unsigned key, bool there) {
            int b = 0;
            const bool mine = there && key >= cut && locate(key_value(key), level, in1, in2, b) && b == bin;
            const unsigned who = __ballot_sync(0xffffffffu, mine);
            if (who == 0u) return;
            const int leader = __ffs(who) - 1;
            unsigned base = 0;
            if (lane == leader) base = atomicAdd(&sh.list_size, (unsigned)__popc(who));
            base = __shfl_sync(0xffffffffu, base, leader);
            if (mine) {
                const unsigned at = base + __popc(who & ((1u << lane) - 1u));
                if (at < (unsigned)kListCapacity) sh.list[at] = key;
            }
        });
        // every block copies the lists of all: what follows runs in each block alone, alike
        cluster_sync();
        unsigned start = 0;
        for (unsigned r = 0; r < blocks; ++r) {
            const unsigned n = peer_u32(&sh.list_size, r);
            for (unsigned i = tid; i < n && start + i < (unsigned)kListCapacity; i += kFilterThreads)
                sh.all[start + i] = peer_u32(&sh.list[i], r);
            start += n;
        }
        if (tid == 0) sh.all_size = min(start, (unsigned)kListCapacity);
        __syncthreads();
    };
    // The kth largest of the kept keys: of the gathered ones (in each block alone), or OF_ROW, of
    // the row (the blocks share it).  Fewer than that many: the smallest possible prefix, which
    // cuts nothing.  Radix selection, a byte a pass.
    auto select_kth_largest = [&](bool of_row, unsigned long long kth) -> unsigned {
        unsigned prefix = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            if (of_row) {
                clear_columns(false);
                each_in_row([&](unsigned key, bool there) {
                    column_add<false>(sh.columns, there && key >= cut && (key & mask) == prefix, (int)((key >> shift) & 255u), 0ull);
                });
                fold_columns(false);
                sum_over_cluster();
            } else {
                clear_sums();
                each_in_all([&](unsigned key, bool) {
                    if (key >= cut && (key & mask) == prefix) atomicAdd(&sh.count[(key >> shift) & 255u], 1u);
                });
                __syncthreads();
            }
            int j;
            unsigned long long above;
            first_crossing<false>([&](int i) { return (unsigned long long)sh.count[255 - i]; }, kth, sh, j, above);
            if (j == 256) {                 // not that many: the lowest byte, everything above it counted
                j = 255;
                above -= sh.count[0];
            }
            prefix |= (unsigned)(255 - j) << shift;
            kth -= above;
        }
        return prefix;
    };
    // The smallest key at which the mass of the kept keys (the gathered ones, or OF_ROW the row's),
    // summed from the smallest key up and starting from `below`, first exceeds `target`.
    auto select_mass_from_below = [&](bool of_row, unsigned long long target, unsigned long long below) -> unsigned {
        unsigned prefix = 0;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            if (of_row) {
                clear_columns(true);
                each_in_row([&](unsigned key, bool there) {
                    const bool in = there && key >= cut && (key & mask) == prefix;
                    column_add<true>(sh.columns, in, (int)((key >> shift) & 255u), in ? fixed_mass(key_value(key), y_max) : 0ull);
                });
                fold_columns(true);
                sum_over_cluster();
            } else {
                clear_sums();
                each_in_all([&](unsigned key, bool) {
                    if (key >= cut && (key & mask) == prefix) add_wide(&sh.mass[(key >> shift) & 255u], fixed_mass(key_value(key), y_max));
                });
                __syncthreads();
            }
            int j;
            unsigned long long before;
            first_crossing<true>([&](int i) { return sh.mass[i]; }, target - below, sh, j, before);
            if (j == 256) {                 // the highest byte holds the first kept token at the latest
                j = 255;
                before -= sh.mass[255];
            }
            prefix |= (unsigned)j << shift;
            below += before;
        }
        return prefix;
    };

    // ---- top-k: the k-th largest key among the kept ones -------------------
    if (k > 0 && k < vocab) {
        unsigned long long need = (unsigned long long)k;        // how many from the top of the bins looked into
        int in1 = 0, in2 = 0;
        unsigned kth = 0;
        bool found = false, fewer = false;
        for (int level = 1; level <= kLevels && !found; ++level) {
            look(level, in1, in2, false);
            int bin;
            unsigned long long above;
            first_crossing<false>([&](int i) { return (unsigned long long)sh.count[i]; }, need, sh, bin, above);
            if (bin == 256) {
                if (level == 1) {           // fewer than k tokens are kept
                    fewer = true;
                    break;
                }
                bin = 255;
                above -= sh.count[255];
            }
            if (level == 1 && bin == kCoarseBins - 1) break;    // the far bin is not divided
            need -= above;
            if (sh.count[bin] <= (unsigned)kListCapacity) {
                gather(level, in1, in2, bin);
                kth = select_kth_largest(false, need);
                found = true;
            } else if (level == 1) {
                in1 = bin;
            } else {
                in2 = bin;
            }
        }
        if (!found && !fewer) kth = select_kth_largest(true, (unsigned long long)k);     // the far bin, or a crowd of near ties
        if (kth > cut) cut = kth;
    }

    // ---- top-p: drop the smallest tokens while their mass stays <= 1 - p ----
    if (p < 1.0f) {
        unsigned long long target = 0, below = 0;
        int in1 = 0, in2 = 0;
        unsigned edge = 0;
        bool found = false;
        for (int level = 1; level <= kLevels && !found; ++level) {
            look(level, in1, in2, true);
            int j;
            unsigned long long before;
            if (level == 1) {
                first_crossing<true>([&](int i) { return sh.mass[i]; }, ~0ull, sh, j, before);   // none crosses: the whole mass
                target = (unsigned long long)((double)before * (double)(1.0f - p));
            }
            first_crossing<true>([&](int i) { return sh.mass[255 - i]; }, target - below, sh, j, before);   // from the smallest up
            if (j == 256) {                 // the bin of the largest tokens holds the first kept one at the latest
                j = 255;
                before -= sh.mass[0];
            }
            const int bin = 255 - j;
            if (level == 1 && bin == kCoarseBins - 1) break;    // the far bin is not divided
            below += before;
            if (sh.count[bin] <= (unsigned)kListCapacity) {
                gather(level, in1, in2, bin);
                edge = select_mass_from_below(false, target, below);
                found = true;
            } else if (level == 1) {
                in1 = bin;
            } else {
                in2 = bin;
            }
        }
        if (!found) edge = select_mass_from_below(true, target, 0ull);
        if (edge > cut) cut = edge;
        const unsigned top_key = ordered_key(y_max);
        if (cut > top_key) cut = top_key;          // the largest token always stays
    }

    // ---- the draw ------------------------------------------------------------
    const unsigned long long seed = seeds[row], draw = draw_index[row];
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int c = (int)rank * kFilterThreads + tid; c < chunks; c += stride) {
        float xs[4];
        load_chunk(c, xs);
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
    best = best_of_cluster(best);
    if (rank == 0 && tid == 0) tokens[row] = best.index == 0x7fffffff ? top.index : best.index;
    cluster_sync();                                // no block leaves while another may read its tables
}

// Penalties on the distinct tokens a request has seen, listed per row in CSR form:
// tokens[offsets[r] .. offsets[r+1]) with the number of times each occurred in the
// output (0 = prompt only).  minivllm/sample/ops/penalties.py:51-72: a seen token's
// logit is divided by the repetition penalty when positive, multiplied when not;
// then frequency * count and presence * [count > 0] are subtracted.
// A row may have one more generated token that the lists do not hold yet, because it is still
// on the device (a step sampled ahead of the one before): last_tokens[last_rows[r]], no such
// token where last_rows[r] is negative.  It counts as if it stood in the lists: one more for a
// listed token, a count of one for a new one, with the arithmetic of a listed token either way.
__global__ void penalties_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ offsets,
                                 const int* __restrict__ seen_tokens, const int* __restrict__ output_counts,
                                 const float* __restrict__ repetition, const float* __restrict__ frequency,
                                 const float* __restrict__ presence, const int* __restrict__ last_tokens,
                                 const int* __restrict__ last_rows) {
    const int row = blockIdx.x;
    float* x = logits + (size_t)row * vocab;
    const float rep = repetition[row], freq = frequency[row], pres = presence[row];
    int last = -1;
    if (last_tokens != nullptr && last_rows[row] >= 0) last = last_tokens[last_rows[row]];
    if (last >= vocab) last = -1;
    auto penalised = [&](float v, int count) {
        v = v > 0.0f ? v * (1.0f / rep) : v * rep;
        v -= freq * (float)count;
        if (count > 0) v -= pres;
        return v;
    };
    bool listed = false;
    for (int i = offsets[row] + threadIdx.x; i < offsets[row + 1]; i += blockDim.x) {
        const int token = seen_tokens[i];
        if (token < 0 || token >= vocab) continue;
        int count = output_counts[i];
        if (token == last) {
            ++count;
            listed = true;
        }
        x[token] = penalised(x[token], count);
    }
    listed = __syncthreads_or(listed);
    if (threadIdx.x == 0 && last >= 0 && !listed) x[last] = penalised(x[last], 1);
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
    if (kinds & 2) {
        static const cudaError_t attribute = cudaFuncSetAttribute(sample_filtered_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                                  (int)sizeof(FilterShared));
        if (attribute != cudaSuccess) return fail("sample", cudaGetErrorString(attribute));
        cudaLaunchConfig_t config = {};
        config.blockDim = dim3(kFilterThreads);
        config.dynamicSmemBytes = sizeof(FilterShared);
        config.stream = stream;
        cudaLaunchAttribute cluster[1];
        cluster[0].id = cudaLaunchAttributeClusterDimension;
        cluster[0].val.clusterDim.y = 1;
        cluster[0].val.clusterDim.z = 1;
        config.attrs = cluster;
        config.numAttrs = 1;
        // Blocks to a row: eight while the GPU then holds all rows at once (a cluster needs its SMs
        // side by side, so fewer clusters of eight fit than an eighth of the SMs), fewer for more rows;
        // never so few that a column of a block could overflow (a thread takes every (blocks * 1024)-th
        // chunk of four tokens, and the 32 warps of a block share a lane's column).
        static int clusters_that_fit[kRowCluster + 1] = {};
        auto fit = [&](int n) {
            if (clusters_that_fit[n] == 0) {
                config.gridDim = dim3(n * 64);
                cluster[0].val.clusterDim.x = n;
                int count = 0;
                if (cudaOccupancyMaxActiveClusters(&count, sample_filtered_kernel, &config) != cudaSuccess || count < 1) {
                    cudaGetLastError();
                    count = sm_count() / (2 * n) > 0 ? sm_count() / (2 * n) : 1;
                }
                clusters_that_fit[n] = count;
            }
            return clusters_that_fit[n];
        };
        auto column_tokens = [&](int n) { return 128ll * ((vocab + 4096ll * n - 1) / (4096ll * n)); };
        int blocks = kRowCluster;
        while (blocks > 2 && rows > fit(blocks)) blocks >>= 1;
        while (blocks < kRowCluster && column_tokens(blocks) > kColumnMaxTokens) blocks <<= 1;
        if (column_tokens(blocks) > kColumnMaxTokens)
            return fail("sample", "filters (top-k, top-p, min-p) take a vocabulary of 1015808 tokens at most");
        config.gridDim = dim3(rows * blocks);
        cluster[0].val.clusterDim.x = blocks;
        cudaLaunchKernelEx(&config, sample_filtered_kernel, logits, vocab, temperature, top_k, top_p, min_p, seeds, draw_index, tokens,
                           greedy_eps);
    }
    return check_launch("sample");
}

// Log-probabilities of the sampled tokens and of the largest tokens of rows that want them (see
// logprobs_kernel); width: columns of ids and values, 1 + the longest list.
B200_EXPORT int b200_logprobs(const float* logits, int rows, int vocab, const int* tokens, const int* wanted, int width,
                              int* ids, float* values, int* place, cudaStream_t stream) {
    using namespace b200;
    if (rows == 0) return 0;
    if (vocab <= 0) return fail("logprobs", "vocabulary must be positive");
    if (width < 1 || width > kMaxLogprobs + 1) return fail("logprobs", "lists of 0 to 32 tokens");
    logprobs_kernel<<<rows * kRowCluster, kLogprobThreads, 0, stream>>>(logits, vocab, tokens, wanted, width, ids, values, place);
    return check_launch("logprobs");
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
                               const float* frequency, const float* presence, const int* last_tokens,
                               const int* last_rows, cudaStream_t stream) {
    // last_tokens / last_rows: null, or per row the place in last_tokens of one more generated token (negative: none)
    using namespace b200;
    if (rows == 0) return 0;
    if ((last_tokens == nullptr) != (last_rows == nullptr)) return fail("penalties", "last tokens and their rows go together");
    penalties_kernel<<<rows, 256, 0, stream>>>(logits, vocab, offsets, seen_tokens, output_counts,
                                               repetition, frequency, presence, last_tokens, last_rows);
    return check_launch("penalties");
}

B200_EXPORT int b200_mask_tokens(float* logits, int vocab, const int* rows, const int* tokens, int count,
                                 cudaStream_t stream) {
    using namespace b200;
    if (count == 0) return 0;
    mask_tokens_kernel<<<(count + 255) / 256, 256, 0, stream>>>(logits, vocab, rows, tokens, count);
    return check_launch("mask_tokens");
}

// Pieces that the kernels on the 5th-generation tensor cores share: a TMA tile load, the shared-memory
// and instruction descriptors of tcgen05.mma for bfloat16 operands in 128-byte-swizzled K-major tiles,
// the MMA and commit instructions, and 16- and 32-column reads of tensor memory.
#pragma once

#include <cuda.h>

#include "async_copy.cuh"

namespace b200 {

constexpr int kTcRows = 128;          // weight rows per block = UMMA M
constexpr int kTcK = 64;              // k elements per stage (one 128-byte swizzle row)
constexpr int kTcATile = kTcRows * kTcK * 2;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile, int byte_offset) {
    const unsigned address = (smem_u32(smem_tile) + byte_offset) & 0x3FFFF;
    unsigned long long desc = 0;
    desc |= (unsigned long long)(address >> 4);                 // start address, 16-byte units
    desc |= (unsigned long long)1 << 16;                        // leading byte offset (unused with swizzle)
    desc |= (unsigned long long)(1024 >> 4) << 32;              // stride byte offset between 8-row groups
    desc |= (unsigned long long)1 << 46;                        // descriptor version of this architecture
    desc |= (unsigned long long)2 << 61;                        // 128-byte swizzle
    return desc;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(kTcRows >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long a, unsigned long long b,
                                          unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"((unsigned)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 columns of this thread's lane of tensor memory; returns when the values are there.
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

}  // namespace b200

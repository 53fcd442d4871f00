// y[M, N] = x[M, K] . w[N, K]^T in IEEE float32 on the CUDA cores: fused
// multiply-add only, no tensor-core mode of reduced precision anywhere.  This is
// every matrix product of the true 32-bit run mode (the reference gets the same
// arithmetic from F.linear with TF32 left off, minivllm/layers/quantization/
// methods.py:36-37).
//
// 64 x 64 output tile per block of 256 threads, 4 x 4 outputs per thread, K in
// slices of 16 staged through shared memory.  Each output sums its K products in
// one fixed order (slice after slice, element after element) whatever M is, so a
// row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace b200 {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x,
                                                       const float* __restrict__ w,
                                                       float* __restrict__ y, int M, int N, int K, int vec_ok) {
    __shared__ __align__(16) float x_s[kTileK][kTileM + 4];
    __shared__ __align__(16) float w_s[kTileK][kTileN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
    const int tx = tid & 15, ty = tid >> 4;             // 16 x 16 threads, each 4 x 4 outputs
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // Loading: 64 rows x 16 k = 1024 elements per operand, 4 per thread.
    const int load_row = tid >> 2;                      // 0..63
    const int load_k = (tid & 3) * 4;                   // 0, 4, 8, 12

    for (int k0 = 0; k0 < K; k0 += kTileK) {
        float xv[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int xm = m0 + load_row, wn = n0 + load_row, kk = k0 + load_k;
        if (xm < M) {
            if (vec_ok && kk + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(x + (size_t)xm * K + kk);
                xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (kk + i < K) xv[i] = x[(size_t)xm * K + kk + i];
            }
        }
        if (wn < N) {
            if (vec_ok && kk + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(w + (size_t)wn * K + kk);
                wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (kk + i < K) wv[i] = w[(size_t)wn * K + kk + i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x_s[load_k + i][load_row] = xv[i];
            w_s[load_k + i][load_row] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTileK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&x_s[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&w_s[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) y[(size_t)m * N + n] = acc[i][j];
        }
    }
}

}  // namespace b200

B200_EXPORT int b200_gemm_f32(const float* x, const float* w, float* y, int M, int N, int K,
                              cudaStream_t stream) {
    using namespace b200;
    if (M == 0 || N == 0) return 0;
    if (M < 0 || N < 0 || K <= 0) return fail("gemm_f32", "sizes must be positive");
    dim3 grid((N + kTileN - 1) / kTileN, (M + kTileM - 1) / kTileM);
    if (grid.y > 65535) return fail("gemm_f32", "more than 65535 * 64 rows in one product");
    // 128-bit loads need rows that start on 16-byte boundaries; otherwise scalar loads.
    const int vec_ok = (K % 4 == 0) && ((((uintptr_t)x | (uintptr_t)w) & 15) == 0);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, y, M, N, K, vec_ok);
    return check_launch("gemm_f32");
}

// True 32-bit matrix product for the float32 path: C[M, N] = A[M, K] * W[N, K]^T with fp32 FMA only
// (no tensor cores, no reduced-precision mode).  Each output element is the sum over k = 0..K-1 in that
// order, so an output row does not depend on M, on the tile it falls in or on the other rows of the batch.
//
// Reference parity: the reference's fp32 product is cublasSgemm (src/ops/kernels/cuda/matmul_kernel.cu:70-88)
// or the plain triple loop on the CPU (include/pulse/ops/kernels/matmul_kernel.hpp:23-35); weights are
// [out, in] and used transposed (src/layer/linear.cpp:213).
#include "common.cuh"

#define TILE_M 64
#define TILE_N 64
#define TILE_K 16

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ A, int lda,
                                                          const float* __restrict__ W, int ldw, float* __restrict__ C,
                                                          int ldc, int M, int N, int K) {
    __shared__ float As[TILE_K][TILE_M + 4];
    __shared__ float Ws[TILE_K][TILE_N + 4];
    pdl_wait();
    pdl_trigger(PDL_PRODUCT);
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each a 4 x 4 patch
    const int m0 = blockIdx.y * TILE_M, n0 = blockIdx.x * TILE_N;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TILE_K) {
        // 64 x 16 elements per operand, 4 per thread; k runs fastest in memory
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = tid + r * 256;
            const int row = idx / TILE_K, kk = idx % TILE_K;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.0f;
            Ws[kk][row] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TILE_K; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}

PI_EXPORT int pi_gemm_f32_nt(const float* A, int lda, const float* W, int ldw, float* C, int ldc, int M, int N, int K,
                             cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return pi_refuse("pi_gemm_f32_nt: K=%d must be positive", K);
    if (lda < K || ldw < K || ldc < N) return pi_refuse("pi_gemm_f32_nt: leading dimensions (%d, %d, %d) too small", lda, ldw, ldc);
    dim3 grid((N + TILE_N - 1) / TILE_N, (M + TILE_M - 1) / TILE_M);
    if (grid.y > 65535) return pi_refuse("pi_gemm_f32_nt: M=%d is beyond the grid limit", M);
    pi_launch(gemm_f32_nt_kernel, grid, dim3(256), 0, stream, A, lda, W, ldw, C, ldc, M, N, K);
    return pi_check_launch("pi_gemm_f32_nt");
}

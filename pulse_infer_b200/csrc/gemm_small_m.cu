// Weight-streaming matrix product for decoding: out[M, N] = x[M, K] * W[N, K]^T in bfloat16 with 32-bit
// accumulation, for a handful of rows (M <= 32).  Every weight is read exactly once, in 16-byte pieces
// that bypass L1, and the product runs on tensor cores with the roles swapped: 16 rows of W are the
// 16-row operand of mma.sync m16n8k16 and 8 rows of x (8 requests) are its 8 columns, so nothing is
// padded along the batch.  The few hundred kilobytes of x stay in L1/L2.
//
// A CTA owns 16 output features; its warps split K into contiguous ranges and their partial sums are added
// in warp order through shared memory, so a result does not depend on the other rows of the batch (for a given
// launch shape; the shape, and with it the split of K, is chosen from M's bucket, N and K).
// Wide outputs (thousands of 16-feature tiles) use 8 warps per CTA with two register sets of weights in
// flight; narrow ones (N = 4096 gives only 256 tiles) use 16 warps per CTA so that the whole GPU still has
// loads in flight.
// (Splitting K further across the CTAs of a thread-block cluster, reduced through distributed shared memory,
// was measured and dropped: it made the 33-100 MB products of a decode step slower, not faster.)
//
// Within a 32-wide block of k, thread t of a quad supplies elements 8t..8t+7 of its row for both operands:
// 8t+0..3 go to the four k slots that the thread owns in the first mma, 8t+4..7 to those of the second.  The
// sum over k does not care which element sits in which slot as long as both operands agree.
//
// Reference parity: the reference calls cublasGemmEx for every product, also at one row
// (src/ops/kernels/cuda/matmul_kernel.cu:132-154); weights are [out, in] and used transposed
// (src/layer/linear.cpp:213).
#include "common.cuh"

#define SM_FEATURES 16      // output features per CTA
#define SM_UNROLL 4         // k blocks in flight per warp

__device__ __forceinline__ uint4 ld_stream16(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                          unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: tiles of 8 rows of x; SM_WARPS: warps per CTA, each takes 1/SM_WARPS of K; DOUBLE: two register sets
// GATED: the 16 rows of W of a CTA are 8 gate features followed by their 8 up features, and the CTA writes
// silu(gate) * up for its 8 features (out has N / 2 columns).
template <int MT, typename TO, int SM_WARPS, bool DOUBLE, int MIN_CTAS, bool GATED>
__global__ void __launch_bounds__(SM_WARPS * 32, MIN_CTAS)
gemm_small_m_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw, TO* __restrict__ out, int ldo,
                    int M, int N, int K) {
    __shared__ float partial[SM_WARPS][SM_FEATURES][MT * 8 + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * SM_FEATURES;

    // rows of W this thread reads (clamped: rows beyond N are computed and dropped)
    const int ra = min(n0 + g, N - 1), rb = min(n0 + g + 8, N - 1);
    const bf16* wa = W + (size_t)ra * ldw + 8 * t;
    const bf16* wb = W + (size_t)rb * ldw + 8 * t;
    const bf16* xr[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) xr[i] = x + (size_t)min(8 * i + g, M - 1) * ldx + 8 * t;

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }

    // 32-wide blocks of k, one contiguous range per warp
    const int blocks = (K + 31) / 32;
    const int per_warp = (blocks + SM_WARPS - 1) / SM_WARPS;
    const int b_begin = warp * per_warp, b_end = min(blocks, b_begin + per_warp);

    // Two register sets of SM_UNROLL blocks each: while one is multiplied the other is in flight.  The first
    // set is requested before pdl_wait(): weights do not depend on the kernel that produces x.
    uint4 va0[SM_UNROLL], vb0[SM_UNROLL];
    auto load_w = [&](int b, uint4 (&va)[SM_UNROLL], uint4 (&vb)[SM_UNROLL]) {
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            const int k = (b + u) * 32 + 8 * t;
            const bool valid = (b + u) < b_end && k + 8 <= K;
            va[u] = valid ? ld_stream16(wa + (size_t)(b + u) * 32) : make_uint4(0, 0, 0, 0);
            vb[u] = valid ? ld_stream16(wb + (size_t)(b + u) * 32) : make_uint4(0, 0, 0, 0);
        }
    };
    auto multiply = [&](int b, const uint4 (&va)[SM_UNROLL], const uint4 (&vb)[SM_UNROLL]) {
#pragma unroll
        for (int u = 0; u < SM_UNROLL; ++u) {
            const int k = (b + u) * 32 + 8 * t;
            const bool valid = (b + u) < b_end && k + 8 <= K;
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const uint4 xv = valid ? __ldg(reinterpret_cast<const uint4*>(xr[i] + (size_t)(b + u) * 32))
                                       : make_uint4(0, 0, 0, 0);
                mma_16816(acc[i], va[u].x, vb[u].x, va[u].y, vb[u].y, xv.x, xv.y);
                mma_16816(acc[i], va[u].z, vb[u].z, va[u].w, vb[u].w, xv.z, xv.w);
            }
        }
    };
    load_w(b_begin, va0, vb0);
    pdl_wait();
    pdl_trigger(PDL_PRODUCT);
    if (DOUBLE) {
        uint4 va1[SM_UNROLL], vb1[SM_UNROLL];
        for (int b = b_begin; b < b_end; b += 2 * SM_UNROLL) {
            load_w(b + SM_UNROLL, va1, vb1);
            multiply(b, va0, vb0);
            load_w(b + 2 * SM_UNROLL, va0, vb0);
            multiply(b + SM_UNROLL, va1, vb1);
        }
    } else {
        for (int b = b_begin; b < b_end; b += SM_UNROLL) {
            multiply(b, va0, vb0);
            load_w(b + SM_UNROLL, va0, vb0);
        }
    }

    // acc[i][0..1]: feature g, rows 8i + 2t, 8i + 2t + 1;  acc[i][2..3]: feature g + 8, same rows
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        partial[warp][g][8 * i + 2 * t] = acc[i][0];
        partial[warp][g][8 * i + 2 * t + 1] = acc[i][1];
        partial[warp][g + 8][8 * i + 2 * t] = acc[i][2];
        partial[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();
    if constexpr (GATED) {
        for (int idx = threadIdx.x; idx < (SM_FEATURES / 2) * MT * 8; idx += SM_WARPS * 32) {
            const int m = idx / (SM_FEATURES / 2), f = idx % (SM_FEATURES / 2);
            if (m >= M || n0 + f + SM_FEATURES / 2 >= N) continue;
            float gate = 0.0f, up = 0.0f;
#pragma unroll
            for (int w = 0; w < SM_WARPS; ++w) { gate += partial[w][f][m]; up += partial[w][f + SM_FEATURES / 2][m]; }
            out[(size_t)m * ldo + n0 / 2 + f] = from_float<TO>(gate / (1.0f + expf(-gate)) * up);
        }
    } else {
        for (int idx = threadIdx.x; idx < SM_FEATURES * MT * 8; idx += SM_WARPS * 32) {
            const int m = idx / SM_FEATURES, f = idx % SM_FEATURES;   // neighbouring threads take neighbouring features
            if (m >= M || n0 + f >= N) continue;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < SM_WARPS; ++w) sum += partial[w][f][m];
            out[(size_t)m * ldo + n0 + f] = from_float<TO>(sum);
        }
    }
}

template <int MT, int WARPS, bool DOUBLE, int MIN_CTAS>
static void launch_small_m_shape(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                 int N, int K, int gated, cudaStream_t stream) {
    const dim3 grid((unsigned)((N + SM_FEATURES - 1) / SM_FEATURES));
    if (gated)     // bf16 output only (checked by the caller)
        pi_launch(gemm_small_m_kernel<MT, bf16, WARPS, DOUBLE, MIN_CTAS, true>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)out, ldo, M, N, K);
    else if (out_dtype == PI_F32)
        pi_launch(gemm_small_m_kernel<MT, float, WARPS, DOUBLE, MIN_CTAS, false>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw, (float*)out, ldo, M, N, K);
    else
        pi_launch(gemm_small_m_kernel<MT, bf16, WARPS, DOUBLE, MIN_CTAS, false>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)out, ldo, M, N, K);
}

// variant 0: chosen from the shape.  1: 8 warps, two register sets, 2 CTAs/SM.  2: 8 warps, two sets, 3 CTAs/SM.
// 3: 16 warps, one set, 2 CTAs/SM (M <= 8 only).  4: 8 warps, one set, 4 CTAs/SM.
template <int MT>
static void launch_small_m(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                           int K, int variant, int gated, cudaStream_t stream) {
    const int tiles = (N + SM_FEATURES - 1) / SM_FEATURES;
    if (variant == 0) {   // from measurements on B200 at the sizes of 8B- to 32B-class models
        if (MT == 1) {
            if (tiles <= 2 * 148) variant = K >= 8192 ? 3 : 1;   // few tiles: deep K wants more warps per tile
            else if (tiles <= 1000) variant = 2;
            else variant = 4;                                    // many waves: light CTAs, four per SM
        } else {
            variant = tiles <= 2 * 148 ? 1 : 2;
        }
    }
    if (variant == 3 && MT != 1) variant = 1;
    switch (variant) {
        case 2: launch_small_m_shape<MT, 8, true, 3>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, gated, stream); break;
        case 3: launch_small_m_shape<1, 16, false, 2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, gated, stream); break;
        case 4: launch_small_m_shape<MT, 8, false, 4>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, gated, stream); break;
        default: launch_small_m_shape<MT, 8, true, 2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, gated, stream); break;
    }
}

PI_EXPORT int pi_gemm_small_m_max_rows() { return 32; }

static int gemm_small_m_impl(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                             int K, int variant, int gated, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 32) return pi_refuse("pi_gemm_small_m: %d rows; this kernel takes at most 32", M);
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
        return pi_refuse("pi_gemm_small_m: K=%d and the leading dimensions (%d, %d) must be positive multiples of 8", K, ldx, ldw);
    if (ldx < K || ldw < K || ldo < (gated ? N / 2 : N)) return pi_refuse("pi_gemm_small_m: leading dimensions (%d, %d, %d) too small", ldx, ldw, ldo);
    if (gated && (out_dtype != PI_BF16 || N % SM_FEATURES != 0))
        return pi_refuse("pi_gemm_small_m: the gated epilogue needs bf16 output and N %% %d == 0 (N=%d)", SM_FEATURES, N);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return pi_refuse("pi_gemm_small_m: operands must be 16-byte aligned");
    if (out_dtype != PI_F32 && out_dtype != PI_BF16) return pi_refuse("pi_gemm_small_m: unknown output dtype code %d", out_dtype);
    if (M <= 8) launch_small_m<1>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, gated, stream);
    else if (M <= 16) launch_small_m<2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, gated, stream);
    else launch_small_m<4>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, gated, stream);
    return pi_check_launch("pi_gemm_small_m");
}

PI_EXPORT int pi_gemm_small_m(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, cudaStream_t stream) {
    return gemm_small_m_impl(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 0, 0, stream);
}

// out[M, N / 2] = silu(x Wg^T) * (x Wu^T) with the rows of W in blocks of 16: 8 gate features, then their 8 up features
PI_EXPORT int pi_gemm_small_m_gated(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K,
                                    cudaStream_t stream) {
    return gemm_small_m_impl(x, ldx, W, ldw, out, PI_BF16, ldo, M, N, K, 0, 1, stream);
}

// the same with the launch shape forced (for measurements)
PI_EXPORT int pi_gemm_small_m_variant(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                      int N, int K, int variant, cudaStream_t stream) {
    return gemm_small_m_impl(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, 0, stream);
}

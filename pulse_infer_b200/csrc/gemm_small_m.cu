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
//
// Within a 32-wide block of k, thread t of a quad supplies elements 8t..8t+7 of its row for both operands:
// 8t+0..3 go to the four k slots that the thread owns in the first mma, 8t+4..7 to those of the second.  The
// sum over k does not care which element sits in which slot as long as both operands agree.
//
// Fused around the product (decoding is a chain of small kernels, and each one costs a few microseconds):
//   EPI_GATED  the 16 rows of W of a CTA are 8 gate features and their 8 up features: out = silu(gate) * up;
//   EPI_RESID  out is the 32-bit residual h and the result is added to it in place (each element has one owner).
//              With `emit` the CTA also prepares the RMSNorm that follows: it writes bf16(h * norm_weight) for its
//              16 features and the sum of h^2 over them, per row, into its own slot of a table of partial sums;
//   row_ssq    the consumer of such a prepared norm: x is bf16(h * norm_weight), and the kernel sums the partial
//              sums in slot order and scales its outputs by rsqrt(mean(h^2) + eps).
// Together they take both norm kernels and the activation kernel out of a decoder layer; the norm's arithmetic
// stays 32-bit, and the order of every sum is fixed.
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
#define EPI_STORE 0
#define EPI_GATED 1     // out[M, N / 2] = silu(gate) * up, rows of W in blocks of 16: 8 gate features, their 8 up features
#define EPI_RESID 2     // out (float) += result
#define SM_MAX_ROWS 32

// what a launch does besides the product
struct SmallMFusion {
    int epilogue;             // EPI_STORE / EPI_GATED / EPI_RESID
    const float* ssq_part;    // [SM_MAX_ROWS][ssq_parts] partial sums of h^2 per row, or null: outputs are scaled by
    int ssq_parts;            //   rsqrt(sum / K + ssq_eps)
    float ssq_eps;
    const void* emit_w;       // EPI_RESID: weight [N] of the norm that follows (bf16, or float if emit_w_f32), or null
    int emit_w_f32;
    bf16* emit_x;             // [M, emit_ldx] <- bf16(h * emit_w)
    int emit_ldx;
    float* emit_part;         // [SM_MAX_ROWS][gridDim.x] <- this CTA's sum of h^2 per row
};

template <int MT, typename TO, int SM_WARPS, bool DOUBLE, int MIN_CTAS, int EPI>
__global__ void __launch_bounds__(SM_WARPS * 32, MIN_CTAS)
gemm_small_m_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw, TO* __restrict__ out, int ldo,
                    int M, int N, int K, const SmallMFusion fu) {
    constexpr bool GATED = EPI == EPI_GATED;
    __shared__ float partial[SM_WARPS][SM_FEATURES][MT * 8 + 1];
    __shared__ float row_scale[MT * 8];
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
    // The scale of each row from a prepared norm, while the first weights are on their way: a warp per row, the
    // partial sums of the row added in a fixed order (lane q takes slots q, q + 32, ...; then the shuffle tree).
    if (fu.ssq_part != nullptr) {
        for (int r = warp; r < MT * 8; r += SM_WARPS) {
            float tot = 0.0f;
            for (int q = lane; q < fu.ssq_parts; q += 32) tot += fu.ssq_part[(size_t)r * fu.ssq_parts + q];
            tot = warp_sum(tot);
            if (lane == 0) row_scale[r] = 1.0f / sqrtf(tot / (float)K + fu.ssq_eps);
        }
    } else if (threadIdx.x < MT * 8) {
        row_scale[threadIdx.x] = 1.0f;
    }
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
            gate *= row_scale[m]; up *= row_scale[m];
            out[(size_t)m * ldo + n0 / 2 + f] = from_float<TO>(gate / (1.0f + expf(-gate)) * up);
        }
    } else {
        // 16 neighbouring threads take the 16 features of a row; whole warps run each pass (16 * MT * 8 is a multiple of 32)
        for (int idx = threadIdx.x; idx < SM_FEATURES * MT * 8; idx += SM_WARPS * 32) {
            const int m = idx / SM_FEATURES, f = idx % SM_FEATURES;
            const bool live = m < M && n0 + f < N;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < SM_WARPS; ++w) sum += partial[w][f][m];
            sum *= row_scale[m];
            if constexpr (EPI == EPI_RESID) {
                float hnew = 0.0f;
                if (live) {
                    TO* dst = out + (size_t)m * ldo + n0 + f;
                    hnew = to_float<TO>(*dst) + sum;
                    *dst = from_float<TO>(hnew);
                }
                if (fu.emit_w != nullptr) {
                    if (live) {
                        const float wn = fu.emit_w_f32 ? reinterpret_cast<const float*>(fu.emit_w)[n0 + f]
                                                       : __bfloat162float(reinterpret_cast<const bf16*>(fu.emit_w)[n0 + f]);
                        fu.emit_x[(size_t)m * fu.emit_ldx + n0 + f] = __float2bfloat16_rn(hnew * wn);
                    }
                    float sq = hnew * hnew;      // 0 for features and rows that do not exist
                    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                    if (f == 0) fu.emit_part[(size_t)m * gridDim.x + blockIdx.x] = sq;
                }
            } else {
                if (live) out[(size_t)m * ldo + n0 + f] = from_float<TO>(sum);
            }
        }
    }
}

template <int MT, int WARPS, bool DOUBLE, int MIN_CTAS>
static void launch_small_m_shape(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                 int N, int K, const SmallMFusion& fu, cudaStream_t stream) {
    const dim3 grid((unsigned)((N + SM_FEATURES - 1) / SM_FEATURES)), block(WARPS * 32);
#define SM_GO(TO, EPI)                                                                                                  \
    pi_launch(gemm_small_m_kernel<MT, TO, WARPS, DOUBLE, MIN_CTAS, EPI>, grid, block, 0, stream, (const bf16*)x, ldx,   \
              (const bf16*)W, ldw, (TO*)out, ldo, M, N, K, fu)
    if (fu.epilogue == EPI_GATED) SM_GO(bf16, EPI_GATED);          // the caller has checked the dtypes
    else if (fu.epilogue == EPI_RESID) SM_GO(float, EPI_RESID);
    else if (out_dtype == PI_F32) SM_GO(float, EPI_STORE);
    else SM_GO(bf16, EPI_STORE);
#undef SM_GO
}

// variant 0: chosen from the shape.  1: 8 warps, two register sets, 2 CTAs/SM.  2: 8 warps, two sets, 3 CTAs/SM.
// 3: 16 warps, one set, 2 CTAs/SM (M <= 8 only).  4: 8 warps, one set, 4 CTAs/SM.
template <int MT>
static void launch_small_m(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                           int K, int variant, const SmallMFusion& fu, cudaStream_t stream) {
    const int tiles = (N + SM_FEATURES - 1) / SM_FEATURES;
    if (variant == 0) {   // from measurements on B200 at the sizes of 8B- to 32B-class models
        const int sms = pi_sm_count();
        if (tiles > 1000) {
            variant = MT == 1 ? 4 : 2;                           // many waves: light CTAs, four per SM (one tile of rows)
        } else {
            // A few waves at most: the shape with the fewest waves (a 449th tile behind 444 resident ones costs a whole
            // second wave), among equals the one with the fewest, heaviest CTAs per SM.
            const int ctas_per_sm[3] = {2, 3, 4}, shape[3] = {1, 2, 4};
            int best_waves = 1 << 30;
            for (int i = 0; i < (MT == 1 ? 3 : 2); ++i) {
                const int waves = (tiles + ctas_per_sm[i] * sms - 1) / (ctas_per_sm[i] * sms);
                if (waves < best_waves) { best_waves = waves; variant = shape[i]; }
            }
            if (MT == 1 && variant == 1 && K >= 8192) variant = 3;   // few tiles and a deep K: more warps per tile
        }
    }
    if (variant == 3 && MT != 1) variant = 1;
    switch (variant) {
        case 2: launch_small_m_shape<MT, 8, true, 3>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, fu, stream); break;
        case 3: launch_small_m_shape<1, 16, false, 2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, fu, stream); break;
        case 4: launch_small_m_shape<MT, 8, false, 4>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, fu, stream); break;
        default: launch_small_m_shape<MT, 8, true, 2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, fu, stream); break;
    }
}

PI_EXPORT int pi_gemm_small_m_max_rows() { return SM_MAX_ROWS; }

static int gemm_small_m_impl(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                             int K, int variant, const SmallMFusion& fu, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > SM_MAX_ROWS) return pi_refuse("pi_gemm_small_m: %d rows; this kernel takes at most %d", M, SM_MAX_ROWS);
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
        return pi_refuse("pi_gemm_small_m: K=%d and the leading dimensions (%d, %d) must be positive multiples of 8", K, ldx, ldw);
    const bool gated = fu.epilogue == EPI_GATED;
    if (ldx < K || ldw < K || ldo < (gated ? N / 2 : N)) return pi_refuse("pi_gemm_small_m: leading dimensions (%d, %d, %d) too small", ldx, ldw, ldo);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return pi_refuse("pi_gemm_small_m: operands must be 16-byte aligned");
    if (out_dtype != PI_F32 && out_dtype != PI_BF16) return pi_refuse("pi_gemm_small_m: unknown output dtype code %d", out_dtype);
    if (fu.epilogue < EPI_STORE || fu.epilogue > EPI_RESID) return pi_refuse("pi_gemm_small_m: unknown epilogue %d", fu.epilogue);
    if (gated && (out_dtype != PI_BF16 || N % SM_FEATURES != 0))
        return pi_refuse("pi_gemm_small_m: the gated epilogue needs bf16 output and N %% %d == 0 (N=%d)", SM_FEATURES, N);
    if (fu.epilogue == EPI_RESID && out_dtype != PI_F32) return pi_refuse("pi_gemm_small_m: the residual epilogue adds to a float32 tensor");
    if (fu.ssq_part != nullptr && fu.ssq_parts <= 0) return pi_refuse("pi_gemm_small_m: %d partial sums", fu.ssq_parts);
    if (fu.emit_w != nullptr && (fu.epilogue != EPI_RESID || fu.emit_x == nullptr || fu.emit_part == nullptr || fu.emit_ldx < N))
        return pi_refuse("pi_gemm_small_m: preparing the next norm goes with the residual epilogue and needs its two outputs");
    if (M <= 8) launch_small_m<1>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, fu, stream);
    else if (M <= 16) launch_small_m<2>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, fu, stream);
    else launch_small_m<4>(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, fu, stream);
    return pi_check_launch("pi_gemm_small_m");
}

static const SmallMFusion kPlain = {EPI_STORE, nullptr, 0, 0.0f, nullptr, 0, nullptr, 0, nullptr};

PI_EXPORT int pi_gemm_small_m(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, cudaStream_t stream) {
    return gemm_small_m_impl(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 0, kPlain, stream);
}

// 16-feature tiles of a product with N outputs = slots of the table of partial sums that `emit` fills
PI_EXPORT int pi_gemm_small_m_tiles(int N) { return (N + SM_FEATURES - 1) / SM_FEATURES; }

// The same with work fused around it.
//   epilogue: 0 store, 1 silu(gate) * up (out [M, N / 2] bf16, rows of W in blocks of 16: 8 gate features, then their 8
//             up features), 2 add to out (float32) in place.
//   ssq_part (or null), ssq_parts, ssq_eps: x is bf16(h * norm_weight) and the outputs are scaled by
//             rsqrt(sum over the ssq_parts slots of ssq_part[row][slot] / K + ssq_eps); 32 rows.
//   emit_w (or null; dtype code emit_w_dtype), emit_x, emit_ldx, emit_part: with epilogue 2, also write
//             emit_x[M, N] = bf16(out * emit_w) and emit_part[row][tile] = sum over the tile's features of out^2
//             (32 rows of pi_gemm_small_m_tiles(N) slots).
PI_EXPORT int pi_gemm_small_m_fused(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                    int N, int K, int epilogue, const float* ssq_part, int ssq_parts, float ssq_eps,
                                    const void* emit_w, int emit_w_dtype, void* emit_x, int emit_ldx, float* emit_part,
                                    cudaStream_t stream) {
    if (emit_w != nullptr && emit_w_dtype != PI_F32 && emit_w_dtype != PI_BF16)
        return pi_refuse("pi_gemm_small_m_fused: unknown dtype code %d of the norm's weight", emit_w_dtype);
    const SmallMFusion fu = {epilogue, ssq_part, ssq_parts, ssq_eps, emit_w, emit_w_dtype == PI_F32 ? 1 : 0, (bf16*)emit_x,
                             emit_ldx, emit_part};
    return gemm_small_m_impl(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, 0, fu, stream);
}

#ifdef PI_MEASURE_HOOKS
// the plain product with the launch shape forced: only in builds made for measurements (-DPI_MEASURE_HOOKS)
PI_EXPORT int pi_gemm_small_m_variant(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M,
                                      int N, int K, int variant, cudaStream_t stream) {
    return gemm_small_m_impl(x, ldx, W, ldw, out, out_dtype, ldo, M, N, K, variant, kPlain, stream);
}
#endif

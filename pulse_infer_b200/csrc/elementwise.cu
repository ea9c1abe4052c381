// Memory-bound kernels of the step: embedding gather, fused residual-add + RMSNorm, SiLU*mul,
// rotation tables, and the fused per-head RMSNorm + rotation + paged key/value write.
//
// Formulas follow the reference engine (paths inside its project):
//   embedding       src/ops/kernels/cuda/embedding_kernel.cu:7-28   (row gather; an id outside the table gives zeros)
//   RMSNorm         src/ops/kernels/cuda/rmsnorm_kernel.cu:97-118,147 (x * rsqrt(mean(x^2) + eps) * w, float math)
//   rotation        src/ops/kernels/cuda/rope_kernel.cu:102-123     (angle = pos / theta^(2i/rot), adjacent pairs)
//   paged write     src/ops/kernels/cuda/paged_kv_write.cu:35-52    (page = table[pos / page], slot = pos % page)
//   SiLU, product   src/ops/kernels/cuda/silu_kernel.cu:78-104, mul_kernel.cu:38-46
// Differences by design: the residual stream is 32-bit, one rounding per fused kernel instead of one per
// reference op, exact expf/sqrtf (the reference builds with fast-math), rotation angles from a table that
// is computed once per step in 64-bit.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------------
// embedding: out[t, :] = table[token[t], :] as 32-bit residual
// ---------------------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, float* __restrict__ out,
                             int hidden, int vocab) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const bool valid = id >= 0 && id < vocab;
    const TW* src = table + (size_t)(valid ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = valid ? to_float<TW>(src[i]) : 0.0f;
}

PI_EXPORT int pi_embed(const int* tokens, const void* table, int table_dtype, float* out, int num_tokens, int hidden,
                       int vocab, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0) return pi_refuse("pi_embed: hidden=%d vocab=%d must be positive", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == PI_BF16)
        pi_launch(embed_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, tokens, (const bf16*)table, out, hidden, vocab);
    else if (table_dtype == PI_F32)
        pi_launch(embed_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, tokens, (const float*)table, out, hidden, vocab);
    else
        return pi_refuse("pi_embed: unknown table dtype code %d", table_dtype);
    return pi_check_launch("pi_embed");
}

// ---------------------------------------------------------------------------------------------------
// fused residual add + RMSNorm
//   rows == nullptr:  h[r] += delta[r] (stored), x[r] = norm(h[r])                    for r in [0, n)
//   rows != nullptr:  x[i] = norm(h[rows[i]] + delta[rows[i]])   (h is left untouched) for i in [0, n)
// One block per row; the sum of squares, the inverse root and the product are 32-bit.
// ---------------------------------------------------------------------------------------------------
template <typename TA, typename TW, int VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TA* __restrict__ delta, const TW* __restrict__ w,
                                   TA* __restrict__ x, const int* __restrict__ rows, int hidden, float eps,
                                   const Prefetch pf) {
    __shared__ float scratch[33];
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const int out_row = blockIdx.x;
    const int src_row = rows ? rows[out_row] : out_row;
    float* hr = h + (size_t)src_row * hidden;
    const TA* dr = delta ? delta + (size_t)src_row * hidden : nullptr;
    TA* xr = x + (size_t)out_row * hidden;
    const bool store_h = (rows == nullptr) && (delta != nullptr);

    float ss = 0.0f;
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
        float v[VEC];
        if (VEC == 4) {
            const float4 hv = *reinterpret_cast<const float4*>(hr + i);
            v[0] = hv.x; v[1 % VEC] = hv.y; v[2 % VEC] = hv.z; v[3 % VEC] = hv.w;
        } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[k] = hr[i + k];
        }
        if (dr) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[k] += to_float<TA>(dr[i + k]);
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss += v[k] * v[k];
        if (store_h) {
            if (VEC == 4) {
                *reinterpret_cast<float4*>(hr + i) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) hr[i + k] = v[k];
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);

    // second pass: every thread re-reads exactly the elements it wrote (or read) above
    const bool readd = (dr != nullptr) && !store_h;
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            float v = hr[i + k];
            if (readd) v += to_float<TA>(dr[i + k]);
            xr[i + k] = from_float<TA>(v * inv * to_float<TW>(w[i + k]));
        }
    }
}

// Same operation with the row held in registers: every load (residual, delta, weight) is issued before
// anything is computed, so a row costs one trip to memory instead of three.  Needs hidden % 4 == 0 and
// hidden <= 256 * 4 * ITEMS.
template <typename TA, typename TW, int ITEMS>
__global__ void __launch_bounds__(256) add_rmsnorm_reg_kernel(float* __restrict__ h, const TA* __restrict__ delta,
                                                              const TW* __restrict__ w, TA* __restrict__ x,
                                                              const int* __restrict__ rows, int hidden, float eps,
                                                              const Prefetch pf) {
    __shared__ float scratch[33];
    struct alignas(sizeof(TA) * 4) PackA { TA v[4]; };
    struct alignas(sizeof(TW) * 4) PackW { TW v[4]; };
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const int out_row = blockIdx.x;
    const int src_row = rows ? rows[out_row] : out_row;
    float* hr = h + (size_t)src_row * hidden;
    const TA* dr = delta ? delta + (size_t)src_row * hidden : nullptr;
    TA* xr = x + (size_t)out_row * hidden;
    const bool store_h = (rows == nullptr) && (delta != nullptr);

    float4 hv[ITEMS];
    PackA dv[ITEMS];
    PackW wv[ITEMS];
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int i = (it * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            hv[it] = *reinterpret_cast<const float4*>(hr + i);
            if (dr) dv[it] = *reinterpret_cast<const PackA*>(dr + i);
            wv[it] = *reinterpret_cast<const PackW*>(w + i);
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int i = (it * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            if (dr) {
                hv[it].x += to_float<TA>(dv[it].v[0]); hv[it].y += to_float<TA>(dv[it].v[1]);
                hv[it].z += to_float<TA>(dv[it].v[2]); hv[it].w += to_float<TA>(dv[it].v[3]);
            }
            ss += hv[it].x * hv[it].x + hv[it].y * hv[it].y + hv[it].z * hv[it].z + hv[it].w * hv[it].w;
            if (store_h) *reinterpret_cast<float4*>(hr + i) = hv[it];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int i = (it * 256 + threadIdx.x) * 4;
        if (i < hidden) {
            PackA o;
            o.v[0] = from_float<TA>(hv[it].x * inv * to_float<TW>(wv[it].v[0]));
            o.v[1] = from_float<TA>(hv[it].y * inv * to_float<TW>(wv[it].v[1]));
            o.v[2] = from_float<TA>(hv[it].z * inv * to_float<TW>(wv[it].v[2]));
            o.v[3] = from_float<TA>(hv[it].w * inv * to_float<TW>(wv[it].v[3]));
            *reinterpret_cast<PackA*>(xr + i) = o;
        }
    }
}

template <typename TA, typename TW>
static void launch_add_rmsnorm(float* h, const void* delta, const void* w, void* x, const int* rows, int n, int hidden,
                               float eps, const Prefetch pf, cudaStream_t stream) {
    const int threads = hidden >= 2048 ? 256 : 128;
    if (hidden % 4 == 0 && hidden <= 256 * 4 * 2)
        pi_launch(add_rmsnorm_reg_kernel<TA, TW, 2>, dim3(n + pi_prefetch_ctas(pf)), dim3(256), 0, stream, h, (const TA*)delta, (const TW*)w, (TA*)x, rows, hidden, eps, pf);
    else if (hidden % 4 == 0 && hidden <= 256 * 4 * 4)
        pi_launch(add_rmsnorm_reg_kernel<TA, TW, 4>, dim3(n + pi_prefetch_ctas(pf)), dim3(256), 0, stream, h, (const TA*)delta, (const TW*)w, (TA*)x, rows, hidden, eps, pf);
    else if (hidden % 4 == 0 && hidden <= 256 * 4 * 8)
        pi_launch(add_rmsnorm_reg_kernel<TA, TW, 8>, dim3(n + pi_prefetch_ctas(pf)), dim3(256), 0, stream, h, (const TA*)delta, (const TW*)w, (TA*)x, rows, hidden, eps, pf);
    else if (hidden % 4 == 0)
        pi_launch(add_rmsnorm_kernel<TA, TW, 4>, dim3(n + pi_prefetch_ctas(pf)), dim3(threads), 0, stream, h, (const TA*)delta, (const TW*)w, (TA*)x, rows, hidden, eps, pf);
    else
        pi_launch(add_rmsnorm_kernel<TA, TW, 1>, dim3(n + pi_prefetch_ctas(pf)), dim3(threads), 0, stream, h, (const TA*)delta, (const TW*)w, (TA*)x, rows, hidden, eps, pf);
}

PI_EXPORT int pi_add_rmsnorm(float* h, const void* delta, const void* weight, int weight_dtype, void* x, int act_dtype,
                             const int* rows, int n, int hidden, float eps, const void* prefetch_ptr,
                             unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (hidden <= 0) return pi_refuse("pi_add_rmsnorm: hidden=%d must be positive", hidden);
    const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, n);
    if (act_dtype == PI_BF16 && weight_dtype == PI_BF16) launch_add_rmsnorm<bf16, bf16>(h, delta, weight, x, rows, n, hidden, eps, pf, stream);
    else if (act_dtype == PI_BF16 && weight_dtype == PI_F32) launch_add_rmsnorm<bf16, float>(h, delta, weight, x, rows, n, hidden, eps, pf, stream);
    else if (act_dtype == PI_F32 && weight_dtype == PI_F32) launch_add_rmsnorm<float, float>(h, delta, weight, x, rows, n, hidden, eps, pf, stream);
    else if (act_dtype == PI_F32 && weight_dtype == PI_BF16) launch_add_rmsnorm<float, bf16>(h, delta, weight, x, rows, n, hidden, eps, pf, stream);
    else return pi_refuse("pi_add_rmsnorm: unknown dtype codes act=%d weight=%d", act_dtype, weight_dtype);
    return pi_check_launch("pi_add_rmsnorm");
}

// ---------------------------------------------------------------------------------------------------
// SiLU(gate) * up on the fused [n, 2*inter] output of the gate_up product: out[n, inter].
// blocked = 0: columns are [all gate | all up].  blocked = 1: columns come in blocks of 16, 8 gate features
// followed by their 8 up features (the layout the products' gated epilogues want of the weight rows).
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total, int blocked,
                                const Prefetch pf) {
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const size_t row = e / inter;
    const int col = (int)(e % inter);
    const int gcol = blocked ? (col / 8) * 16 + col % 8 : col;
    const int ucol = blocked ? gcol + 8 : inter + col;
    const float g = to_float<T>(gu[row * 2 * (size_t)inter + gcol]);
    const float u = to_float<T>(gu[row * 2 * (size_t)inter + ucol]);
    out[e] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// 8 elements (bf16) or 4 (float) per thread with 16-byte accesses; needs inter % VEC == 0
template <typename T, int VEC>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, size_t total_vecs,
                                    int blocked, const Prefetch pf) {
    struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_vecs) return;
    const int vecs_per_row = inter / VEC;
    const size_t row = idx / vecs_per_row;
    const int col = (int)(idx % vecs_per_row) * VEC;
    const int gcol = blocked ? (col / 8) * 16 + col % 8 : col;       // VEC divides 8: a vector stays inside a block
    const int ucol = blocked ? gcol + 8 : inter + col;
    const Pack g = *reinterpret_cast<const Pack*>(gu + row * 2 * (size_t)inter + gcol);
    const Pack u = *reinterpret_cast<const Pack*>(gu + row * 2 * (size_t)inter + ucol);
    Pack o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const float gv = to_float<T>(g.v[k]);
        o.v[k] = from_float<T>(gv / (1.0f + expf(-gv)) * to_float<T>(u.v[k]));
    }
    *reinterpret_cast<Pack*>(out + row * (size_t)inter + col) = o;
}

PI_EXPORT int pi_silu_mul(const void* gate_up, void* out, int dtype, int n, int inter, int blocked, const void* prefetch_ptr,
                          unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (inter <= 0) return pi_refuse("pi_silu_mul: inter=%d must be positive", inter);
    if (blocked && inter % 8 != 0) return pi_refuse("pi_silu_mul: the blocked layout needs inter %% 8 == 0 (inter=%d)", inter);
    const size_t total = (size_t)n * inter;
    const int threads = 256;
    if (dtype == PI_BF16 && inter % 8 == 0) {
        const size_t vecs = total / 8;
        const unsigned own = (unsigned)((vecs + threads - 1) / threads);
        const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, (int)own);
        pi_launch(silu_mul_vec_kernel<bf16, 8>, dim3(own + pi_prefetch_ctas(pf)), dim3(threads), 0, stream,
                  (const bf16*)gate_up, (bf16*)out, inter, vecs, blocked, pf);
    } else if (dtype == PI_F32 && inter % 4 == 0) {
        const size_t vecs = total / 4;
        const unsigned own = (unsigned)((vecs + threads - 1) / threads);
        const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, (int)own);
        pi_launch(silu_mul_vec_kernel<float, 4>, dim3(own + pi_prefetch_ctas(pf)), dim3(threads), 0, stream,
                  (const float*)gate_up, (float*)out, inter, vecs, blocked, pf);
    } else if (dtype == PI_BF16 || dtype == PI_F32) {
        // widths that are no multiple of the vector: rows may start unaligned, so plain element accesses
        const unsigned blocks = (unsigned)((total + threads - 1) / threads);
        const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, (int)blocks);
        if (dtype == PI_BF16) pi_launch(silu_mul_kernel<bf16>, dim3(blocks + pi_prefetch_ctas(pf)), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, total, blocked, pf);
        else pi_launch(silu_mul_kernel<float>, dim3(blocks + pi_prefetch_ctas(pf)), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, total, blocked, pf);
    } else {
        return pi_refuse("pi_silu_mul: unknown dtype code %d", dtype);
    }
    return pi_check_launch("pi_silu_mul");
}

// ---------------------------------------------------------------------------------------------------
// rotation tables for one step: cos/sin of pos[t] / divisor[i], angle in 64-bit, stored as 32-bit
// ---------------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ divisors,
                                  float* __restrict__ cos_out, float* __restrict__ sin_out, int num_tokens, int pairs) {
    pdl_wait();
    pdl_trigger();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= num_tokens * pairs) return;
    const int t = idx / pairs, i = idx % pairs;
    const double angle = (double)positions[t] / divisors[i];
    double s, c;
    sincos(angle, &s, &c);
    cos_out[idx] = (float)c;
    sin_out[idx] = (float)s;
}

PI_EXPORT int pi_rope_table(const int* positions, const double* divisors, float* cos_out, float* sin_out, int num_tokens,
                            int pairs, cudaStream_t stream) {
    if (num_tokens <= 0 || pairs <= 0) return 0;
    const int total = num_tokens * pairs, threads = 128;
    pi_launch(rope_table_kernel, dim3((total + threads - 1) / threads), dim3(threads), 0, stream, positions, divisors, cos_out,
              sin_out, num_tokens, pairs);
    return pi_check_launch("pi_rope_table");
}

// ---------------------------------------------------------------------------------------------------
// fused per-head RMSNorm + rotation + paged key/value write.
// Input: qkv [T, row_stride] holding nq query heads, then nkv key heads, then nkv value heads, each of width d.
// One warp per (token, head):
//   query head: normalise (weight qw), rotate, write back in place
//   key head:   normalise (weight kw), rotate, write into K page
//   value head: copy into V page
// pairing: 1 = adjacent pairs (2i, 2i+1) as the reference computes; 0 = split halves (i, i + rot/2).
// Elements at and beyond rot (partial rotation) are normalised but not rotated.
// A token whose page id is negative is skipped and counted in *error_count.
// ---------------------------------------------------------------------------------------------------
#define QK_MAX_PAIRS 4  // pairs per lane: head_dim up to 256

template <typename TA, typename TW>
__global__ void qk_norm_rope_write_kernel(TA* __restrict__ qkv, int row_stride, const TW* __restrict__ qw,
                                          const TW* __restrict__ kw, float eps, int has_norm,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_pairs,
                                          int adjacent, TA* __restrict__ kcache, TA* __restrict__ vcache,
                                          const int* __restrict__ block_table, int bt_stride,
                                          const int* __restrict__ token_slot, const int* __restrict__ positions,
                                          int page_size, int nq, int nkv, int d, int* __restrict__ error_count,
                                          const Prefetch pf) {
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    if (head >= nq + 2 * nkv) return;
    TA* src = qkv + (size_t)t * row_stride + (size_t)head * d;

    TA* dst = src;  // query heads are rewritten in place
    if (head >= nq) {
        const int kvh = (head - nq) % nkv;
        const int pos = positions[t];
        const int page = block_table[(size_t)token_slot[t] * bt_stride + pos / page_size];
        if (page < 0) {
            if (lane == 0) atomicAdd(error_count, 1);
            return;
        }
        TA* base = (head < nq + nkv) ? kcache : vcache;
        dst = base + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * d;
    }

    // 16-bit activations whose rows and heads start on 8-byte boundaries move in 8-byte pieces
    const bool wide = sizeof(TA) == 2 && (d & 3) == 0 && (row_stride & 3) == 0 && ((uintptr_t)qkv & 7) == 0 &&
                      ((uintptr_t)kcache & 7) == 0 && ((uintptr_t)vcache & 7) == 0;
    if (head >= nq + nkv) {  // value head: plain copy
        if (wide) {
            for (int e = lane; e < d / 4; e += 32) reinterpret_cast<uint2*>(dst)[e] = reinterpret_cast<const uint2*>(src)[e];
        } else {
            for (int e = lane; e < d; e += 32) dst[e] = src[e];
        }
        return;
    }

    const TW* w = head < nq ? qw : kw;
    if (sizeof(TA) == 2 && wide && adjacent) {
        // a lane takes two adjacent pairs (four elements) at a time: the same arithmetic as below, wider accesses
        const bf16* s16 = reinterpret_cast<const bf16*>(src);
        bf16* d16 = reinterpret_cast<bf16*>(dst);
        constexpr int QUADS = QK_MAX_PAIRS / 2;
        float x[QUADS][4];
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < QUADS; ++k) {
            const int qd = lane + 32 * k;
#pragma unroll
            for (int i = 0; i < 4; ++i) x[k][i] = 0.0f;
            if (qd < d / 4) {
                const uint2 raw = reinterpret_cast<const uint2*>(s16)[qd];
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                x[k][0] = __low2float(a); x[k][1] = __high2float(a); x[k][2] = __low2float(b); x[k][3] = __high2float(b);
                ss += x[k][0] * x[k][0] + x[k][1] * x[k][1];
                ss += x[k][2] * x[k][2] + x[k][3] * x[k][3];
            }
        }
        float inv = 1.0f;
        if (has_norm) {
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)d + eps);
        }
        __syncwarp();
#pragma unroll
        for (int k = 0; k < QUADS; ++k) {
            const int qd = lane + 32 * k;
            if (qd < d / 4) {
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = has_norm ? x[k][i] * inv * to_float<TW>(w[4 * qd + i]) : x[k][i];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int p = 2 * qd + h;
                    if (p < rot_pairs) {
                        const float c = cos_t[(size_t)t * rot_pairs + p], sn = sin_t[(size_t)t * rot_pairs + p];
                        const float r0 = v[2 * h] * c - v[2 * h + 1] * sn;
                        const float r1 = v[2 * h] * sn + v[2 * h + 1] * c;
                        v[2 * h] = r0; v[2 * h + 1] = r1;
                    }
                }
                const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
                uint2 raw;
                raw.x = *reinterpret_cast<const unsigned*>(&a); raw.y = *reinterpret_cast<const unsigned*>(&b);
                reinterpret_cast<uint2*>(d16)[qd] = raw;
            }
        }
        return;
    }
    const int half_pairs = d / 2;
    float x0[QK_MAX_PAIRS], x1[QK_MAX_PAIRS];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < QK_MAX_PAIRS; ++k) {
        const int p = lane + 32 * k;
        x0[k] = 0.0f; x1[k] = 0.0f;
        if (p < half_pairs) {
            int i0, i1;
            if (p < rot_pairs && !adjacent) { i0 = p; i1 = p + rot_pairs; }
            else { i0 = 2 * p; i1 = 2 * p + 1; }
            x0[k] = to_float<TA>(src[i0]);
            x1[k] = to_float<TA>(src[i1]);
            ss += x0[k] * x0[k] + x1[k] * x1[k];
        }
    }
    float inv = 1.0f;
    if (has_norm) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)d + eps);
    }
    // all loads of this head are done before any store (in-place rewrite of query heads)
    __syncwarp();
#pragma unroll
    for (int k = 0; k < QK_MAX_PAIRS; ++k) {
        const int p = lane + 32 * k;
        if (p < half_pairs) {
            int i0, i1;
            if (p < rot_pairs && !adjacent) { i0 = p; i1 = p + rot_pairs; }
            else { i0 = 2 * p; i1 = 2 * p + 1; }
            float v0 = x0[k], v1 = x1[k];
            if (has_norm) {
                v0 = v0 * inv * to_float<TW>(w[i0]);
                v1 = v1 * inv * to_float<TW>(w[i1]);
            }
            if (p < rot_pairs) {
                const float c = cos_t[(size_t)t * rot_pairs + p], s = sin_t[(size_t)t * rot_pairs + p];
                const float r0 = v0 * c - v1 * s;
                const float r1 = v0 * s + v1 * c;
                v0 = r0; v1 = r1;
            }
            dst[i0] = from_float<TA>(v0);
            dst[i1] = from_float<TA>(v1);
        }
    }
}

// The same for the common case - bfloat16 activations, adjacent pairs, head size up to 128 and a multiple of 8, a number
// of rotated pairs that is a multiple of 4, everything on 16-byte boundaries.  The general kernel is bound neither by
// memory bandwidth nor by arithmetic: a 2,048-token portion takes it 30 us at 10 % of DRAM bandwidth, because a lane
// has one 8-byte load in flight at a time (Little's law: 64 warps x 256 B per SM and microsecond are 16 GB/s).  Here a
// lane takes eight elements (four adjacent pairs) of a head with 16-byte loads, so a warp works on two heads at once,
// and on QK_FAST_UNROLL such pairs of heads per pass with all their loads issued before the first use; a fixed number
// of blocks walks the (token, head) pairs.  The arithmetic and its order per element are those of the general kernel
// (the sum of squares is added in another order).
#ifndef QK_FAST_UNROLL
#define QK_FAST_UNROLL 2
#endif

template <typename TW>
__global__ void qk_norm_rope_write_fast_kernel(bf16* __restrict__ qkv, int row_stride, const TW* __restrict__ qw,
                                               const TW* __restrict__ kw, float eps, int has_norm,
                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_pairs,
                                               bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                                               const int* __restrict__ block_table, int bt_stride,
                                               const int* __restrict__ token_slot, const int* __restrict__ positions,
                                               int page_size, int nq, int nkv, int d, int num_tokens,
                                               int* __restrict__ error_count, const Prefetch pf) {
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    constexpr int U = QK_FAST_UNROLL;
    const int lane = threadIdx.x & 31, half = lane >> 4, sub = lane & 15;
    const int heads = nq + 2 * nkv;
    const int own_blocks = pf.bytes ? pf.first_cta : (int)gridDim.x;
    const int total = num_tokens * heads;              // the launcher has checked that this fits
    const int per_pass = 2 * U;                        // (token, head) pairs a warp takes per pass
    const int stride = own_blocks * (int)(blockDim.x >> 5) * per_pass;
    const bool mine = 8 * sub < d;
    for (int first = ((int)blockIdx.x * (int)(blockDim.x >> 5) + (int)(threadIdx.x >> 5)) * per_pass; first < total; first += stride) {
        uint4 raw[U];
        bf16* dst[U];
        int tok[U], hd[U];
        bool live[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int unit = first + 2 * j + half;
            live[j] = unit < total;
            const int t = live[j] ? unit / heads : 0;
            const int head = live[j] ? unit - t * heads : 0;
            tok[j] = t; hd[j] = head;
            bf16* src = qkv + (size_t)t * row_stride + head * d;
            dst[j] = src;                                // query heads are rewritten in place
            if (live[j] && head >= nq) {
                const int kvh = head - nq - (head >= nq + nkv ? nkv : 0);
                const int pos = positions[t];
                const int page_index = pos / page_size;
                const int page = block_table[(size_t)token_slot[t] * bt_stride + page_index];
                if (page < 0) {
                    if (sub == 0) atomicAdd(error_count, 1);
                    live[j] = false;
                } else {
                    bf16* base = (head < nq + nkv) ? kcache : vcache;
                    dst[j] = base + (((size_t)page * nkv + kvh) * page_size + (pos - page_index * page_size)) * d;
                }
            }
            raw[j] = (live[j] && mine) ? reinterpret_cast<const uint4*>(src)[sub] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int head = hd[j];
            float x[8];
            {
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) { x[2 * i] = __low2float(h2[i]); x[2 * i + 1] = __high2float(h2[i]); }
            }
            // the sum of squares over the 16 lanes of the head (every lane of the warp takes part; lanes without
            // elements hold zeros)
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i += 2) ss += x[i] * x[i] + x[i + 1] * x[i + 1];
            ss += __shfl_xor_sync(0xffffffffu, ss, 8);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            if (!live[j] || !mine) continue;
            if (head >= nq + nkv) {                      // value head: plain copy
                reinterpret_cast<uint4*>(dst[j])[sub] = raw[j];
                continue;
            }
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = x[i];
            if (has_norm) {
                const TW* w = head < nq ? qw : kw;
                float wv[8];
                if constexpr (sizeof(TW) == 2) {
                    const uint4 wr = reinterpret_cast<const uint4*>(w)[sub];
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { wv[2 * i] = __low2float(h2[i]); wv[2 * i + 1] = __high2float(h2[i]); }
                } else {
                    const float4 w0 = reinterpret_cast<const float4*>(w)[2 * sub], w1 = reinterpret_cast<const float4*>(w)[2 * sub + 1];
                    wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                }
                const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = x[i] * inv * wv[i];
            }
            if (4 * sub < rot_pairs) {                   // rot_pairs is a multiple of 4: all four pairs of the lane rotate, or none
                const float4 c = reinterpret_cast<const float4*>(cos_t + (size_t)tok[j] * rot_pairs)[sub];
                const float4 sn = reinterpret_cast<const float4*>(sin_t + (size_t)tok[j] * rot_pairs)[sub];
                const float cs[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float r0 = v[2 * h] * cs[h] - v[2 * h + 1] * ss4[h];
                    const float r1 = v[2 * h] * ss4[h] + v[2 * h + 1] * cs[h];
                    v[2 * h] = r0; v[2 * h + 1] = r1;
                }
            }
            uint4 out;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            reinterpret_cast<uint4*>(dst[j])[sub] = out;
        }
    }
}

PI_EXPORT int pi_qk_norm_rope_write(void* qkv, int row_stride, int act_dtype, const void* q_weight, const void* k_weight,
                                    int weight_dtype, float eps, int has_norm, const float* cos_t, const float* sin_t,
                                    int rot_pairs, int adjacent, void* kcache, void* vcache, const int* block_table,
                                    int bt_stride, const int* token_slot, const int* positions, int page_size, int nq,
                                    int nkv, int d, int num_tokens, int* error_count, const void* prefetch_ptr,
                                    unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (d <= 0 || d % 2 != 0 || d > 64 * QK_MAX_PAIRS)
        return pi_refuse("pi_qk_norm_rope_write: head_dim=%d must be even and at most %d", d, 64 * QK_MAX_PAIRS);
    if (rot_pairs < 0 || rot_pairs * 2 > d) return pi_refuse("pi_qk_norm_rope_write: rotary width %d exceeds head_dim %d", rot_pairs * 2, d);
    if (nq < 0 || nkv < 0 || nq + nkv == 0) return pi_refuse("pi_qk_norm_rope_write: nq=%d nkv=%d", nq, nkv);
    if (nkv > 0 && page_size <= 0) return pi_refuse("pi_qk_norm_rope_write: page_size=%d must be positive", page_size);
    const int warps = 4;
    const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, num_tokens);
    dim3 grid(num_tokens + pi_prefetch_ctas(pf), (nq + 2 * nkv + warps - 1) / warps);
    // the common case on the kernel with few instructions per head (see above); everything else on the general one
    const bool aligned16 = (((uintptr_t)qkv | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)q_weight | (uintptr_t)k_weight |
                             (uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0;
    if (act_dtype == PI_BF16 && adjacent && d % 8 == 0 && d <= 128 && row_stride % 8 == 0 && rot_pairs % 4 == 0 && aligned16 &&
        (weight_dtype == PI_BF16 || weight_dtype == PI_F32) && (long long)num_tokens * (nq + 2 * nkv) < (1LL << 30)) {
        const int fast_warps = 8;
        const long long units = (long long)num_tokens * (nq + 2 * nkv);
        long long blocks = (units + fast_warps * 2 * QK_FAST_UNROLL - 1) / (fast_warps * 2 * QK_FAST_UNROLL);
        const long long most = (long long)pi_sm_count() * 8;          // eight blocks of eight warps fill an SM
        if (blocks > most) blocks = most;
        const Prefetch pf_fast = pi_make_prefetch(prefetch_ptr, prefetch_bytes, (int)blocks);
        const dim3 fgrid((unsigned)(blocks + pi_prefetch_ctas(pf_fast)));
        if (weight_dtype == PI_BF16)
            pi_launch(qk_norm_rope_write_fast_kernel<bf16>, fgrid, dim3(fast_warps * 32), 0, stream, (bf16*)qkv, row_stride,
                      (const bf16*)q_weight, (const bf16*)k_weight, eps, has_norm, cos_t, sin_t, rot_pairs, (bf16*)kcache,
                      (bf16*)vcache, block_table, bt_stride, token_slot, positions, page_size, nq, nkv, d, num_tokens,
                      error_count, pf_fast);
        else
            pi_launch(qk_norm_rope_write_fast_kernel<float>, fgrid, dim3(fast_warps * 32), 0, stream, (bf16*)qkv, row_stride,
                      (const float*)q_weight, (const float*)k_weight, eps, has_norm, cos_t, sin_t, rot_pairs, (bf16*)kcache,
                      (bf16*)vcache, block_table, bt_stride, token_slot, positions, page_size, nq, nkv, d, num_tokens,
                      error_count, pf_fast);
        return pi_check_launch("pi_qk_norm_rope_write");
    }
#define QK_LAUNCH(TA, TW)                                                                                              \
    pi_launch(qk_norm_rope_write_kernel<TA, TW>, grid, dim3(warps * 32), 0, stream,                                      \
        (TA*)qkv, row_stride, (const TW*)q_weight, (const TW*)k_weight, eps, has_norm, cos_t, sin_t, rot_pairs, adjacent, \
        (TA*)kcache, (TA*)vcache, block_table, bt_stride, token_slot, positions, page_size, nq, nkv, d, error_count, pf)
    if (act_dtype == PI_BF16 && weight_dtype == PI_BF16) QK_LAUNCH(bf16, bf16);
    else if (act_dtype == PI_BF16 && weight_dtype == PI_F32) QK_LAUNCH(bf16, float);
    else if (act_dtype == PI_F32 && weight_dtype == PI_F32) QK_LAUNCH(float, float);
    else if (act_dtype == PI_F32 && weight_dtype == PI_BF16) QK_LAUNCH(float, bf16);
    else return pi_refuse("pi_qk_norm_rope_write: unknown dtype codes act=%d weight=%d", act_dtype, weight_dtype);
#undef QK_LAUNCH
    return pi_check_launch("pi_qk_norm_rope_write");
}

// Paged attention, plain version: one warp per (query token, query head), keys visited in order in groups
// of 32 with a running maximum and sum (online softmax), everything in 32-bit.  It takes any head size up
// to 256, any number of heads and groups, any page size, an optional window, and both float and bfloat16
// storage.  It is the attention of the float32 path and the cross-check of the tensor-core kernel.
//
// Reference parity: src/ops/kernels/cuda/paged_attention.cu:65-137 — kv head = head / (nq / nkv), score =
// (q . k) * rsqrt(d) over keys 0..pos of the token's own request, causal by the token's absolute position,
// running max / sum / accumulator update per key, out = acc / sum.
// The window (keys pos - window + 1 .. pos) has no counterpart there.
#include <math.h>

#include "common.cuh"

#define SIMPLE_WARPS 4
#define SIMPLE_MAX_CHUNKS 8  // head_dim up to 256

template <typename T>
__global__ void attn_simple_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ kcache,
                                   const T* __restrict__ vcache, const int* __restrict__ block_table, int bt_stride,
                                   const int* __restrict__ token_slot, const int* __restrict__ positions,
                                   T* __restrict__ out, int nq, int nkv, int d, int page_size, int window, float scale) {
    extern __shared__ float qs_all[];  // [SIMPLE_WARPS][d]
    pdl_wait();
    pdl_trigger(PDL_ATTENTION);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * SIMPLE_WARPS + warp;
    if (head >= nq) return;  // whole warp leaves; no block-wide barrier below
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int slot = token_slot[t];
    const int kvh = head / (nq / nkv);
    const int* table = block_table + (size_t)slot * bt_stride;

    float* qs = qs_all + warp * d;
    const T* qrow = q + (size_t)t * q_stride + (size_t)head * d;
    for (int e = lane; e < d; e += 32) qs[e] = to_float<T>(qrow[e]);
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[SIMPLE_MAX_CHUNKS];
#pragma unroll
    for (int i = 0; i < SIMPLE_MAX_CHUNKS; ++i) acc[i] = 0.0f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        int page = -1;
        float s = -INFINITY;
        if (valid) {
            page = table[j / page_size];
            if (page >= 0) {
                const T* krow = kcache + (((size_t)page * nkv + kvh) * page_size + (j % page_size)) * d;
                float dot = 0.0f;
                for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_float<T>(krow[e]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float base = (m_new == -INFINITY) ? 0.0f : m_new;
        const float alpha = expf(m - base);      // m = -inf gives 0
        const float p = expf(s - base);          // s = -inf gives 0
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < SIMPLE_MAX_CHUNKS; ++i) acc[i] *= alpha;
        const int count = (pos - j0 + 1) < 32 ? (pos - j0 + 1) : 32;
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int pg = __shfl_sync(0xffffffffu, page, jj);
            if (pg < 0) continue;
            const int jk = j0 + jj;
            const T* vrow = vcache + (((size_t)pg * nkv + kvh) * page_size + (jk % page_size)) * d;
#pragma unroll
            for (int i = 0; i < SIMPLE_MAX_CHUNKS; ++i) {
                const int e = lane + 32 * i;
                if (e < d) acc[i] = fmaf(pj, to_float<T>(vrow[e]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * nq * d + (size_t)head * d;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < SIMPLE_MAX_CHUNKS; ++i) {
        const int e = lane + 32 * i;
        if (e < d) orow[e] = from_float<T>(acc[i] * inv);
    }
}

PI_EXPORT int pi_attention_simple(const void* q, int q_stride, const void* kcache, const void* vcache, int dtype,
                                  const int* block_table, int bt_stride, const int* token_slot, const int* positions,
                                  void* out, int num_tokens, int nq, int nkv, int d, int page_size, int window,
                                  float scale, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (d <= 0 || d > 32 * SIMPLE_MAX_CHUNKS) return pi_refuse("pi_attention_simple: head_dim=%d must be in 1..%d", d, 32 * SIMPLE_MAX_CHUNKS);
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) return pi_refuse("pi_attention_simple: nq=%d must be a positive multiple of nkv=%d", nq, nkv);
    if (page_size <= 0) return pi_refuse("pi_attention_simple: page_size=%d must be positive", page_size);
    dim3 grid(num_tokens, (nq + SIMPLE_WARPS - 1) / SIMPLE_WARPS);
    if (grid.y > 65535) return pi_refuse("pi_attention_simple: too many heads (%d)", nq);
    const size_t smem = (size_t)SIMPLE_WARPS * d * sizeof(float);
    if (dtype == PI_F32)
        pi_launch(attn_simple_kernel<float>, grid, dim3(SIMPLE_WARPS * 32), smem, stream,
            (const float*)q, q_stride, (const float*)kcache, (const float*)vcache, block_table, bt_stride, token_slot,
            positions, (float*)out, nq, nkv, d, page_size, window, scale);
    else if (dtype == PI_BF16)
        pi_launch(attn_simple_kernel<bf16>, grid, dim3(SIMPLE_WARPS * 32), smem, stream,
            (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, block_table, bt_stride, token_slot,
            positions, (bf16*)out, nq, nkv, d, page_size, window, scale);
    else
        return pi_refuse("pi_attention_simple: unknown dtype code %d", dtype);
    return pi_check_launch("pi_attention_simple");
}

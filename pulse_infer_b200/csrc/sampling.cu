// Token selection on the device from 32-bit logits: greedy (argmax) and temperature sampling with
// optional top-k and top-p, one thread block per row, plus a small kernel that edits single logits
// (presence penalty, banned ids).
//
// Reference parity (the reference samples on the CPU):
//   greedy       src/scheduler/continuous_batch_engine.cpp:20-62   strict '>' so the lowest index wins ties
//   temperature  demo/qwen3_infer.cpp:382-393   weight = exp((logit - max) / temperature); <= 0 means greedy
//   top-k        demo/qwen3_infer.cpp:336-358   the k largest; among equal logits the earlier index stays
//   top-p        demo/qwen3_infer.cpp:395-409   shortest prefix (by descending logit) with cumulative mass >= p
//   draw         demo/qwen3_infer.cpp:411-422   uniform in [0, total), first candidate with cumulative >= draw
//   penalty/ban  demo/qwen3_infer.cpp:251-264, 522-535
// Differences by design: the draw comes from a counter-based generator keyed by (seed, draw index) so a
// request's tokens do not depend on batching; the cumulative walk is in index order rather than sorted
// order (the distribution is the same); all logits equal to the top-p threshold are kept.
#include <limits.h>
#include <math.h>

#include "common.cuh"

__device__ __forceinline__ unsigned ordered_key(float f) {
    // monotone map float -> unsigned (NaN sorts lowest so it is never chosen)
    if (f != f) return 0u;
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// uniform in [0, 1) with 24 bits, from (seed, counter)
__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long counter) {
    const unsigned long long r = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull));
    return (float)(r >> 40) * (1.0f / 16777216.0f);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgMax block_argmax(const float* __restrict__ x, int n, ArgMax* sh /* 33 */) {
    ArgMax best = {-INFINITY, -1};
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = x[i];
        if (v == v && (best.i < 0 || v > best.v)) { best.v = v; best.i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other;
        other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < nwarps ? sh[lane] : ArgMax{-INFINITY, -1};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other;
            other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, other);
        }
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    const ArgMax r = sh[32];
    __syncthreads();
    return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int ld, int vocab, int* __restrict__ out) {
    __shared__ ArgMax sh[33];
    pdl_wait();
    pdl_trigger();
    const ArgMax r = block_argmax(logits + (size_t)blockIdx.x * ld, vocab, sh);
    if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

// Large vocabularies: a row is cut into slices scanned by separate blocks (one block per row would leave
// most of the GPU idle and take tens of microseconds), then one small block per row picks among the slices.
#define ARGMAX_SLICE 4096
__global__ void argmax_slices_kernel(const float* __restrict__ logits, int ld, int vocab, float* __restrict__ cand_val,
                                     int* __restrict__ cand_idx, int slices) {
    __shared__ ArgMax sh[33];
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.y, slice = blockIdx.x;
    const int begin = slice * ARGMAX_SLICE;
    const int n = min(ARGMAX_SLICE, vocab - begin);
    ArgMax r = block_argmax(logits + (size_t)row * ld + begin, n, sh);
    if (threadIdx.x == 0) {
        cand_val[row * slices + slice] = r.v;
        cand_idx[row * slices + slice] = r.i < 0 ? -1 : r.i + begin;
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx, int slices,
                                   int* __restrict__ out) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    ArgMax best = {-INFINITY, -1};
    for (int i = threadIdx.x; i < slices; i += 32) {   // ascending index per lane; ties keep the lower index
        ArgMax c = {cand_val[row * slices + i], cand_idx[row * slices + i]};
        best = better(best, c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other;
        other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
        best = better(best, other);
    }
    if (threadIdx.x == 0) out[row] = best.i;
}

PI_EXPORT int pi_argmax_scratch_floats(int rows, int vocab) {
    const int slices = (vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
    return vocab >= 4 * ARGMAX_SLICE ? 2 * rows * slices : 0;
}

// scratch: pi_argmax_scratch_floats(rows, vocab) 4-byte words (may be null when that is 0)
PI_EXPORT int pi_argmax(const float* logits, int ld, int rows, int vocab, int* out, void* scratch, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return pi_refuse("pi_argmax: vocab=%d ld=%d", vocab, ld);
    if (vocab >= 4 * ARGMAX_SLICE) {
        if (scratch == nullptr) return pi_refuse("pi_argmax: scratch is missing");
        if (rows > 65535) return pi_refuse("pi_argmax: %d rows are beyond the grid limit", rows);
        const int slices = (vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
        float* cand_val = (float*)scratch;
        int* cand_idx = (int*)scratch + (size_t)rows * slices;
        pi_launch(argmax_slices_kernel, dim3(slices, rows), dim3(256), 0, stream, logits, ld, vocab, cand_val, cand_idx, slices);
        pi_launch(argmax_pick_kernel, dim3(rows), dim3(32), 0, stream, (const float*)cand_val, (const int*)cand_idx, slices, out);
    } else {
        pi_launch(argmax_kernel, dim3(rows), dim3(vocab >= 4096 ? 1024 : 256), 0, stream, logits, ld, vocab, out);
    }
    return pi_check_launch("pi_argmax");
}

// exclusive scan over the block in thread order; returns the exclusive prefix, *total gets the sum
template <typename T>
__device__ T block_exclusive_scan(T v, T* sh /* 33 */, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    T incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        T w = lane < nwarps ? sh[lane] : (T)0;
        T wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const T n = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += n;
        }
        sh[lane] = wi - w;  // exclusive prefix of the warps
        if (lane == 31) sh[32] = wi;
    }
    __syncthreads();
    const T result = sh[warp] + (incl - v);
    *total = sh[32];
    __syncthreads();
    return result;
}

__global__ void sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
                              const int* __restrict__ top_k, const float* __restrict__ top_p,
                              const unsigned long long* __restrict__ seeds,
                              const unsigned long long* __restrict__ counters, int* __restrict__ out,
                              const long long* __restrict__ row_entry) {
    __shared__ ArgMax sh_arg[33];
    __shared__ float sh_f[33];
    __shared__ int sh_i[33];
    __shared__ int sh_pick;
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * ld;
    const ArgMax top = block_argmax(x, vocab, sh_arg);
    // Without row_entry the options of row r sit at index r.  With it, row_entry[2r] names the entry of the option
    // tables that row r uses (tables filled once per set of options) and row_entry[2r + 1] is its draw counter.
    const int entry = row_entry != nullptr ? (int)row_entry[2 * row] : row;
    const unsigned long long counter = row_entry != nullptr ? (unsigned long long)row_entry[2 * row + 1] : counters[row];
    const float temp = temperature[entry];
    if (temp <= 0.0f || top.i < 0) {
        if (threadIdx.x == 0) out[row] = top.i;
        return;
    }
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int c0 = threadIdx.x * chunk, c1 = min(vocab, c0 + chunk);

    // ---- top-k: the key of the k-th largest logit, and up to which index equal logits are kept ----------
    const int k = top_k[entry];
    unsigned key_k = 0u;       // keep keys > key_k, and keys == key_k with index <= tie_cut
    int tie_cut = INT_MAX;
    if (k > 0 && k < vocab) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_k | (1u << bit);
            float cnt = 0.0f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) cnt += ordered_key(x[i]) >= cand ? 1.0f : 0.0f;
            cnt = block_sum(cnt, sh_f);  // counts up to 2^24 are exact in float
            if (cnt >= (float)k) key_k = cand;
        }
        float gt = 0.0f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) gt += ordered_key(x[i]) > key_k ? 1.0f : 0.0f;
        const int ties_allowed = k - (int)block_sum(gt, sh_f);
        int mine = 0;
        for (int i = c0; i < c1; ++i) mine += ordered_key(x[i]) == key_k;
        int total_ties;
        const int before = block_exclusive_scan<int>(mine, sh_i, &total_ties);
        if (threadIdx.x == 0) sh_pick = INT_MAX;
        __syncthreads();
        if (ties_allowed < total_ties && before < ties_allowed && before + mine >= ties_allowed) {
            int seen = before;
            for (int i = c0; i < c1; ++i)
                if (ordered_key(x[i]) == key_k && ++seen == ties_allowed) { sh_pick = i; break; }
        }
        __syncthreads();
        tie_cut = sh_pick;
        __syncthreads();
    }
    // key 0 is NaN only; with no top-k, key_k stays 0 and every number is kept
    auto kept_k = [&](int i, unsigned key) { return key != 0u && (key > key_k || (key == key_k && i <= tie_cut)); };
    const float inv_t = 1.0f / temp;

    // ---- top-p: the largest value v whose upper mass (logit >= v, inside the top-k set) reaches p * Z ---
    const float pp = top_p[entry];
    unsigned key_p = 0u;
    if (pp > 0.0f && pp < 1.0f) {
        float z = 0.0f;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            if (kept_k(i, ordered_key(x[i]))) z += expf((x[i] - top.v) * inv_t);
        z = block_sum(z, sh_f);
        const float want = pp * z;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_p | (1u << bit);
            float mass = 0.0f;
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const unsigned key = ordered_key(x[i]);
                if (key >= cand && kept_k(i, key)) mass += expf((x[i] - top.v) * inv_t);
            }
            mass = block_sum(mass, sh_f);
            if (mass >= want) key_p = cand;
        }
    }

    // ---- draw: first index (in index order) whose cumulative kept weight reaches u * total --------------
    float mine = 0.0f;
    int last_kept = -1;
    for (int i = c0; i < c1; ++i) {
        const unsigned key = ordered_key(x[i]);
        if (key >= key_p && kept_k(i, key)) { mine += expf((x[i] - top.v) * inv_t); last_kept = i; }
    }
    float total;
    const float before = block_exclusive_scan<float>(mine, sh_f, &total);
    const float target = uniform_from(seeds[entry], counter) * total;
    if (threadIdx.x == 0) sh_pick = INT_MAX;
    __syncthreads();
    int pick = INT_MAX;
    if (last_kept >= 0 && before + mine >= target) {
        float run = before;
        pick = last_kept;
        for (int i = c0; i < c1; ++i) {
            const unsigned key = ordered_key(x[i]);
            if (key >= key_p && kept_k(i, key)) {
                run += expf((x[i] - top.v) * inv_t);
                if (run >= target) { pick = i; break; }
            }
        }
    }
    if (pick != INT_MAX) atomicMin(&sh_pick, pick);
    __syncthreads();
    int result = sh_pick;
    __syncthreads();
    if (result == INT_MAX) {  // rounding left the target beyond every prefix: take the last kept index
        if (threadIdx.x == 0) sh_pick = -1;
        __syncthreads();
        if (last_kept >= 0) atomicMax(&sh_pick, last_kept);
        __syncthreads();
        result = sh_pick;
    }
    if (threadIdx.x == 0) out[row] = result;
}

PI_EXPORT int pi_sample(const float* logits, int ld, int rows, int vocab, const float* temperature, const int* top_k,
                        const float* top_p, const unsigned long long* seeds, const unsigned long long* counters,
                        int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return pi_refuse("pi_sample: vocab=%d ld=%d", vocab, ld);
    if (vocab > (1 << 24)) return pi_refuse("pi_sample: vocab=%d is beyond 2^24", vocab);
    pi_launch(sample_kernel, dim3(rows), dim3(vocab >= 4096 ? 1024 : 256), 0, stream, logits, ld, vocab, temperature, top_k,
              top_p, seeds, counters, out, (const long long*)nullptr);
    return pi_check_launch("pi_sample");
}

// The same with the options in tables of `entries` entries that outlive the step: row r uses entry row_entry[2r]
// and draw counter row_entry[2r + 1] (int64 pairs: the only per-step data, one small copy).
PI_EXPORT int pi_sample_entries(const float* logits, int ld, int rows, int vocab, const float* temperature, const int* top_k,
                                const float* top_p, const unsigned long long* seeds, const long long* row_entry,
                                int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0 || ld < vocab) return pi_refuse("pi_sample_entries: vocab=%d ld=%d", vocab, ld);
    if (vocab > (1 << 24)) return pi_refuse("pi_sample_entries: vocab=%d is beyond 2^24", vocab);
    if (row_entry == nullptr) return pi_refuse("pi_sample_entries: the (entry, counter) pairs are missing");
    pi_launch(sample_kernel, dim3(rows), dim3(vocab >= 4096 ? 1024 : 256), 0, stream, logits, ld, vocab, temperature, top_k,
              top_p, seeds, (const unsigned long long*)nullptr, out, row_entry);
    return pi_check_launch("pi_sample_entries");
}

// logits[rows[i], tokens[i]] = set ? values[i] : logits[...] + values[i]; (row, token) pairs must be distinct
__global__ void logit_edit_kernel(float* __restrict__ logits, int ld, int vocab, const int* __restrict__ rows,
                                  const int* __restrict__ tokens, const float* __restrict__ values, int n, int set) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int tok = tokens[i];
    if (tok < 0 || tok >= vocab) return;
    float* dst = logits + (size_t)rows[i] * ld + tok;
    *dst = set ? values[i] : *dst + values[i];
}

PI_EXPORT int pi_logit_edit(float* logits, int ld, int vocab, const int* rows, const int* tokens, const float* values,
                            int n, int set, cudaStream_t stream) {
    if (n <= 0) return 0;
    pi_launch(logit_edit_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, logits, ld, vocab, rows, tokens, values, n, set);
    return pi_check_launch("pi_logit_edit");
}

// Paged attention on tensor cores for bfloat16: one kernel body for prompt portions (many query rows,
// all keys) and for decoding (few query rows, keys split across warps and across CTAs).
//
// Rows of a tile are (token, head-in-group) pairs of ONE kv head of ONE request segment, so a key/value
// tile fetched through the block table is shared by all query heads of the group.  S = Q K^T and
// O += P V run on mma.sync m16n8k16 (bf16 in, fp32 accumulate); the running maximum, the sums and the
// rescaling are 32-bit (online softmax, exp2 of scores pre-multiplied by log2(e)/sqrt(d)).  Keys and
// values arrive in shared memory by 16-byte cp.async through the page table, two or three tiles deep.
//
//   prompt mode  (ROW_WARPS x 1 warps): each warp owns 16 rows and walks every key tile.
//   decode mode  (1 x KEY_WARPS warps): the warps share 16 rows and each takes a quarter of every key
//                tile; blockIdx.z additionally splits the keys into ranges of `split_keys`; partial
//                (max, sum, accumulator) triples are merged in shared memory, and across CTAs by
//                attn_merge_kernel.  The number of ranges depends on the request's own length only.
//
// The head size is a compile-time constant (PI_HEAD_DIM, a multiple of 16 up to 256); the library is
// built once per head size a model needs.
//
// Reference parity: src/ops/kernels/cuda/paged_attention.cu:65-137 (grouping, scale, causal bound by
// absolute position, online softmax, out = acc / sum, pages with a negative id are skipped).
#include <math.h>

#include "attention_noalloc.h"
#include "common.cuh"

#ifndef PI_HEAD_DIM
#error "compile with -DPI_HEAD_DIM=<multiple of 16>"
#endif
static_assert(PI_HEAD_DIM % 16 == 0 && PI_HEAD_DIM >= 16 && PI_HEAD_DIM <= 256, "head size must be 16..256 in steps of 16");

#define BN 64  // keys per tile

struct AttnParams {
    const bf16* q;        // [T, q_stride] query heads (already normalised and rotated)
    int q_stride;
    const bf16* kcache;   // [pages, nkv, page_size, D]
    const bf16* vcache;
    const int* block_table;  // [slots, bt_stride]
    int bt_stride;
    const int* seg_off;    // [segments] first token (row of q/out) of the segment
    const int* seg_slot;   // [segments] row of the block table
    const int* seg_start;  // [segments] absolute position of the segment's first token
    const int* seg_len;    // [segments] number of tokens
    bf16* out;             // [T, nq * D]
    float* part_acc;       // [T * nq, max_splits, D] unnormalised partial outputs (decode mode)
    float* part_ml;        // [T * nq, max_splits, 2] (max in log2 units, sum)
    int max_splits;
    int nq, nkv, group;
    int page_size;
    int window;            // 0: all keys
    float scale_log2;      // log2(e) / sqrt(D)
    int tiles_per_seg;
    int num_segments;
    int split_keys;        // keys per range in decode mode (a multiple of BN)
    int decode;            // 1: handle segments of one token only; 0: handle the others only
};

// first key a query at `pos` sees, rounded down to a tile boundary, and the number of key ranges
__device__ __forceinline__ int window_lo(int pos, int window) {
    return (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
}
__device__ __forceinline__ int decode_num_splits(int pos, int window, int split_keys) {
    const int lo_al = (window_lo(pos, window) / BN) * BN;
    return (pos + 1 - lo_al + split_keys - 1) / split_keys;
}
// The ranges a kernel really cuts a request into: never more than the scratch has room for.  When the caller's
// bound is smaller than the request needs, the last range runs on to the newest key, so every key is still read
// exactly once and no partial result is written beyond the scratch.
__device__ __forceinline__ int decode_ranges(int pos, int window, int split_keys, int max_splits) {
    const int n = decode_num_splits(pos, window, split_keys);
    return n < max_splits ? n : max_splits;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x (low half) = lo
    return *reinterpret_cast<unsigned*>(&v);
}

template <int D, int ROW_WARPS, int KEY_WARPS, int STAGES>
__global__ void __launch_bounds__(ROW_WARPS* KEY_WARPS * 32) attn_mma_kernel(const AttnParams p) {
    constexpr int BM = ROW_WARPS * 16;
    constexpr int NTHREADS = ROW_WARPS * KEY_WARPS * 32;
    constexpr int LDS = D + 8;              // padded row length in elements: conflict-free ldmatrix
    constexpr int CHUNKS = D / 8;           // 16-byte chunks per row
    constexpr int KPW = BN / KEY_WARPS;     // keys of a tile that one warp handles
    static_assert(STAGES == 2 || STAGES == 3, "two or three stages");
    static_assert(KPW % 16 == 0, "a warp needs whole k16 steps");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                  // [BM][LDS]
    bf16* Ks = Qs + BM * LDS;                                      // [STAGES][BN][LDS]
    bf16* Vs = Ks + STAGES * BN * LDS;                             // [STAGES][BN][LDS]

    pdl_wait();
    pdl_trigger(PDL_ATTENTION);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wr = warp / KEY_WARPS, wk = warp % KEY_WARPS;
    // Prompt mode: a linear grid ordered so that, for every kv head in turn, the tiles with the most keys (the
    // last rows of a portion) start first; the light tiles fill the tail.  Decode mode: (row tile, kv head, range).
    int seg, tile, kvh, split;
    if (KEY_WARPS == 1) {
        kvh = blockIdx.x % p.nkv;
        const int rest = blockIdx.x / p.nkv;
        tile = p.tiles_per_seg - 1 - rest / p.num_segments;
        seg = rest % p.num_segments;
        split = 0;
    } else {
        seg = blockIdx.x / p.tiles_per_seg;
        tile = blockIdx.x % p.tiles_per_seg;
        kvh = blockIdx.y;
        split = blockIdx.z;
    }

    const int len = p.seg_len[seg];
    if ((len == 1) != (p.decode != 0)) return;
    const int G = p.group;
    const int rows_total = len * G;
    const int row0 = tile * BM;
    if (row0 >= rows_total) return;
    const int start = p.seg_start[seg];
    const int tok_off = p.seg_off[seg];
    const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.bt_stride;

    const int row_last = (row0 + BM < rows_total ? row0 + BM : rows_total) - 1;
    const int pos_first = start + row0 / G, pos_last = start + row_last / G;
    // key range of this CTA: [kbegin, kend), kbegin on a tile boundary
    int kbegin = (window_lo(pos_first, p.window) / BN) * BN;
    int kend = pos_last + 1;
    int nsplits = 1;
    if (p.decode) {
        nsplits = decode_ranges(pos_first, p.window, p.split_keys, p.max_splits);
        if (split >= nsplits) return;
        kbegin += split * p.split_keys;
        if (split + 1 < nsplits && kbegin + p.split_keys < kend) kend = kbegin + p.split_keys;
    } else if (split > 0) {
        return;
    }
    const int num_tiles = (kend - kbegin + BN - 1) / BN;

    // ---- loaders -----------------------------------------------------------------------------------
    auto load_q = [&]() {
        for (int idx = tid; idx < BM * CHUNKS; idx += NTHREADS) {
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            const int rf = row0 + r;
            const bool valid = rf < rows_total;
            const int tok = valid ? rf / G : 0, h = valid ? rf % G : 0;
            const bf16* src = p.q + (size_t)(tok_off + tok) * p.q_stride + (size_t)(kvh * G + h) * D + c * 8;
            cp_async16(Qs + r * LDS + c * 8, src, valid);
        }
    };
    // Element offset of every key row of a tile inside the page pools, looked up through the block table by
    // the first BN threads one tile ahead of the copies that use it (so neither the table lookup nor the
    // divisions sit on the critical path); ~0 marks a row that does not exist.
    __shared__ size_t row_off[2][BN];
    static_assert(NTHREADS >= BN, "the first BN threads fill the row-offset table");
    auto compute_rows = [&](int kt, int buf) {
        if (tid < BN) {
            const int j = kbegin + kt * BN + tid;
            size_t off = ~(size_t)0;
            if (kt < num_tiles && j < kend) {
                const int page = table[j / p.page_size];
                if (page >= 0) off = (((size_t)page * p.nkv + kvh) * p.page_size + (j % p.page_size)) * D;
            }
            row_off[buf][tid] = off;
        }
    };
    auto load_kv = [&](int kt, int stage) {
        bf16* kd = Ks + stage * BN * LDS;
        bf16* vd = Vs + stage * BN * LDS;
        const size_t* offs = row_off[kt & 1];
#pragma unroll
        for (int idx = tid; idx < BN * CHUNKS; idx += NTHREADS) {
            const int r = idx / CHUNKS, c = idx % CHUNKS;
            const size_t off = offs[r];
            const bool valid = off != ~(size_t)0;
            const size_t src = valid ? off + c * 8 : 0;
            cp_async16(kd + r * LDS + c * 8, p.kcache + src, valid);
            cp_async16(vd + r * LDS + c * 8, p.vcache + src, valid);
        }
    };

    // ---- per-thread row bookkeeping ------------------------------------------------------------------
    const int g = lane >> 2, tq = lane & 3;
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int rf = row0 + wr * 16 + g + 8 * i;
        if (rf < rows_total) {
            pos_r[i] = start + rf / G;
            lo_r[i] = window_lo(pos_r[i], p.window);
        } else {
            pos_r[i] = -1;  // no key is visible
            lo_r[i] = 0;
        }
    }
    // visibility bounds of the whole warp (uniform): used to skip tiles
    const int wrow_first = row0 + wr * 16;
    int warp_pos_max = -1, warp_lo_min = 0;
    int warp_pos_min = -1, warp_lo_max = 0;   // a key range inside [warp_lo_max, warp_pos_min] needs no mask
    if (wrow_first < rows_total) {
        const int wrow_last = (wrow_first + 15 < rows_total ? wrow_first + 15 : rows_total - 1);
        warp_pos_max = start + wrow_last / G;
        warp_lo_min = window_lo(start + wrow_first / G, p.window);
        if (wrow_first + 15 < rows_total) {   // all 16 rows exist
            warp_pos_min = start + wrow_first / G;
            warp_lo_max = window_lo(warp_pos_max, p.window);
        }
    }

    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = 0.0f; o[i][1] = 0.0f; o[i][2] = 0.0f; o[i][3] = 0.0f; }

    // ---- pipeline ------------------------------------------------------------------------------------
    // Tile t is copied STAGES-1 iterations before it is used; its row offsets are computed one iteration
    // before that, into half (t & 1) of the table, which the copies of tile t-2 were the last to read.
#pragma unroll
    for (int t = 0; t < STAGES - 1; ++t) compute_rows(t, t & 1);
    __syncthreads();
    load_q();
#pragma unroll
    for (int t = 0; t < STAGES - 1; ++t) {
        if (t < num_tiles) load_kv(t, t);
        cp_async_commit();
    }
    if (STAGES == 3) __syncthreads();  // half 0 is about to be rewritten
    compute_rows(STAGES - 1, (STAGES - 1) & 1);

    for (int kt = 0; kt < num_tiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();  // tile kt (and Q) visible to all; everyone is done with the stage refilled below
        if (kt + STAGES - 1 < num_tiles) load_kv(kt + STAGES - 1, (kt + STAGES - 1) % STAGES);
        cp_async_commit();
        compute_rows(kt + STAGES, (kt + STAGES) & 1);

        const int stage = kt % STAGES;
        const bf16* ks = Ks + stage * BN * LDS;
        const bf16* vs = Vs + stage * BN * LDS;
        const int kw0 = kbegin + kt * BN + wk * KPW;  // first key of this warp's share
        if (kw0 > warp_pos_max || kw0 + KPW - 1 < warp_lo_min) continue;  // nothing visible (uniform per warp)

        // S = Q K^T for 16 rows x KPW keys
        float s[KPW / 8][4];
#pragma unroll
        for (int i = 0; i < KPW / 8; ++i) { s[i][0] = 0.0f; s[i][1] = 0.0f; s[i][2] = 0.0f; s[i][3] = 0.0f; }
#pragma unroll
        for (int ks16 = 0; ks16 < D / 16; ++ks16) {
            unsigned a[4];
            ldmatrix_x4(a, Qs + (wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks16 * 16 + 8 * (lane >> 4));
#pragma unroll
            for (int np = 0; np < KPW / 16; ++np) {
                unsigned b[4];
                ldmatrix_x4(b, ks + (wk * KPW + np * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks16 * 16 + 8 * ((lane >> 3) & 1));
                mma_bf16(s[2 * np], a, b[0], b[1]);
                mma_bf16(s[2 * np + 1], a, b[2], b[3]);
            }
        }

        // mask, scale, running maximum
        float mx[2] = {-INFINITY, -INFINITY};
        if (kw0 >= warp_lo_max && kw0 + KPW - 1 <= warp_pos_min && kw0 + KPW <= kend) {
            // every key of this share is visible to every row of the warp
#pragma unroll
            for (int nt = 0; nt < KPW / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = s[nt][e] * p.scale_log2;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < KPW / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int j = kw0 + nt * 8 + 2 * tq + (e & 1);
                    const bool visible = j <= pos_r[i] && j >= lo_r[i] && j < kend;
                    const float v = visible ? s[nt][e] * p.scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
            }
        }
        float alpha[2], base[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_r[i], mx[i]);
            base[i] = (m_new == -INFINITY) ? 0.0f : m_new;
            alpha[i] = exp2f(m_r[i] - base[i]);
            m_r[i] = m_new;
        }
        float rs[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nt = 0; nt < KPW / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f(s[nt][e] - base[e >> 1]);
                s[nt][e] = pv;
                rs[e >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) l_r[i] = l_r[i] * alpha[i] + rs[i];  // quad partial; summed at the end
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0];
            o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
        }

        // O += P V
#pragma unroll
        for (int kp = 0; kp < KPW / 16; ++kp) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
            a[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
            a[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
            a[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                unsigned b[4];
                ldmatrix_x4_trans(b, vs + (wk * KPW + kp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + dp * 16 + 8 * (lane >> 4));
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();

    // quad-wide sums
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 1);
        l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 2);
    }

    if (KEY_WARPS == 1) {
        // each warp owns its rows: write them out (prompt mode never splits)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int rf = row0 + wr * 16 + g + 8 * i;
            if (rf >= rows_total) continue;
            const int tok = rf / G, h = rf % G;
            const float inv = l_r[i] > 0.0f ? 1.0f / l_r[i] : 0.0f;
            bf16* orow = p.out + (size_t)(tok_off + tok) * p.nq * D + (size_t)(kvh * G + h) * D;
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt)
                *reinterpret_cast<unsigned*>(orow + dt * 8 + 2 * tq) = pack_bf16(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
        }
        return;
    }

    // decode mode: merge the KEY_WARPS partial results of the 16 shared rows through shared memory
    __syncthreads();  // everyone is done reading K/V tiles
    float* mo = reinterpret_cast<float*>(Ks);        // [KEY_WARPS][16][D]
    float* mm = mo + KEY_WARPS * 16 * D;             // [KEY_WARPS][16]
    float* ml = mm + KEY_WARPS * 16;                 // [KEY_WARPS][16]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        float* dst = mo + (wk * 16 + r) * D;
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) {
            dst[dt * 8 + 2 * tq] = o[dt][2 * i];
            dst[dt * 8 + 2 * tq + 1] = o[dt][2 * i + 1];
        }
        if (tq == 0) { mm[wk * 16 + r] = m_r[i]; ml[wk * 16 + r] = l_r[i]; }
    }
    __syncthreads();
    const int valid_rows = rows_total - row0 < 16 ? rows_total - row0 : 16;
    for (int idx = tid; idx < valid_rows * D; idx += NTHREADS) {
        const int r = idx / D, e = idx % D;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < KEY_WARPS; ++w) mstar = fmaxf(mstar, mm[w * 16 + r]);
        float lsum = 0.0f, acc = 0.0f;
        if (mstar != -INFINITY) {
#pragma unroll
            for (int w = 0; w < KEY_WARPS; ++w) {
                const float f = exp2f(mm[w * 16 + r] - mstar);
                lsum += ml[w * 16 + r] * f;
                acc += mo[(w * 16 + r) * D + e] * f;
            }
        }
        const int rf = row0 + r;
        const int tok = rf / G, h = rf % G;
        const size_t orow = (size_t)(tok_off + tok) * p.nq + (size_t)(kvh * G + h);
        if (nsplits == 1) {
            p.out[orow * D + e] = __float2bfloat16_rn(lsum > 0.0f ? acc / lsum : 0.0f);
        } else {
            p.part_acc[(orow * p.max_splits + split) * D + e] = acc;
            if (e == 0) {
                p.part_ml[(orow * p.max_splits + split) * 2] = mstar;
                p.part_ml[(orow * p.max_splits + split) * 2 + 1] = lsum;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Decoding, second form: one new token per request, so a (request, kv head) has only G = nq / nkv query
// rows.  Here the operands are swapped: the 16-row side of the mma holds 16 KEYS and the 8-column side
// holds the query rows (no padding of 4 rows to 16, half the accumulator registers, half the mma count):
//     S^T[key, row] = K[key, :] . Q[row, :]         A = K slice (16 keys x d),   B = Q^T
//     O^T[dim, row] += V^T[dim, key] P^T[key, row]  A = V^T (ldmatrix.trans),    B = P^T (movmatrix of S^T)
// K goes from global memory straight into A fragments (16-byte loads; the d index is permuted inside
// 32-wide blocks, identically for K and Q, which a dot product does not notice); only V is staged in shared
// memory, per warp, by cp.async three slices deep.  The four warps of a CTA take the 16-key slices of the
// CTA's key range in turn and never wait for one another until the final merge, so 16 warps per SM keep
// loads in flight.  Needs D % 32 == 0 and G <= 8 * NT.
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint4 ldg_stream16(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// CONTIG: the page size is a multiple of 16, so the 16 keys of a slice are 16 consecutive rows of one page and a
// slice needs one table lookup and no exchange of offsets between lanes.
template <int D, int NT, bool CONTIG>
__global__ void __launch_bounds__(128, (D * NT <= 128) ? 4 : 2) attn_decode_kernel(const AttnParams p) {
    constexpr int LDS = D + 8;
    constexpr int CHUNKS = D / 8;
    constexpr int DB = D / 32;             // 32-wide blocks of d
    constexpr int VSTAGES = 3;
    constexpr int WARPS = 4;
    static_assert(D % 32 == 0, "this kernel takes head sizes that are multiples of 32");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_wait();
    pdl_trigger(PDL_ATTENTION);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int seg = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    if (p.seg_len[seg] != 1) return;
    const int G = p.group;
    const int pos = p.seg_start[seg];
    const int tok = p.seg_off[seg];
    const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.bt_stride;
    const int lo = window_lo(pos, p.window);
    const int nsplits = decode_ranges(pos, p.window, p.split_keys, p.max_splits);
    if (split >= nsplits) return;
    const int kbegin = (lo / BN) * BN + split * p.split_keys;
    const int kend = split + 1 < nsplits ? min(pos + 1, kbegin + p.split_keys) : pos + 1;
    const int nslices = (kend - kbegin + 15) / 16;

    bf16* vs = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * VSTAGES * 16 * LDS;   // this warp's V stages

    // ---- Q as B fragments: row 8*nt + g, elements 32*db + 8*t .. +7 -------------------------------------
    uint4 qf[NT][DB];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int r = 8 * nt + g;
        const bf16* qrow = p.q + (size_t)tok * p.q_stride + (size_t)(kvh * G + (r < G ? r : 0)) * D + 8 * t;
#pragma unroll
        for (int db = 0; db < DB; ++db)
            qf[nt][db] = r < G ? *reinterpret_cast<const uint4*>(qrow + 32 * db) : make_uint4(0, 0, 0, 0);
    }

    // ---- per-slice helpers ---------------------------------------------------------------------------------
    // What a lane keeps about a slice: CONTIG - the element offset of the slice's first key (same in every lane);
    // otherwise - the offset of key (lane & 15), exchanged by shuffles when rows are addressed.  ~0: no such key.
    auto slice_offsets = [&](int slice) -> size_t {
        const int j = kbegin + 16 * slice + (CONTIG ? 0 : (lane & 15));
        size_t off = ~(size_t)0;
        if (slice < nslices && j < kend) {
            const int page = table[j / p.page_size];
            if (page >= 0) off = (((size_t)page * p.nkv + kvh) * p.page_size + (j % p.page_size)) * D;
        }
        return off;
    };
    auto offset_of_row = [&](size_t mine, int row) -> size_t {
        if (CONTIG) return mine == ~(size_t)0 ? mine : mine + (size_t)row * D;
        const unsigned lo32 = __shfl_sync(0xffffffffu, (unsigned)(mine & 0xffffffffu), row);
        const unsigned hi32 = __shfl_sync(0xffffffffu, (unsigned)(mine >> 32), row);
        return ((size_t)hi32 << 32) | lo32;
    };
    auto load_v = [&](size_t mine, int slice, int stage) {      // 16 rows x CHUNKS 16-byte pieces, 32 lanes
        bf16* dst = vs + stage * 16 * LDS;
        const int rows_valid = kend - (kbegin + 16 * slice);     // rows beyond the range are zero-filled
#pragma unroll
        for (int c = 0; c < (16 * CHUNKS) / 32; ++c) {
            const int idx = lane + 32 * c;
            const int r = idx / CHUNKS, ch = idx % CHUNKS;
            const size_t off = offset_of_row(mine, r);
            const bool valid = off != ~(size_t)0 && r < rows_valid;
            cp_async16(dst + r * LDS + ch * 8, p.vcache + (valid ? off + ch * 8 : 0), valid);
        }
    };
    auto load_k = [&](size_t mine, uint4 (&ka)[DB], uint4 (&kb)[DB]) {   // keys g and g + 8 of the slice
        // rows beyond the range but inside the page hold old finite data; their scores are masked below
        const size_t oa = offset_of_row(mine, g), ob = offset_of_row(mine, g + 8);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
            ka[db] = oa != ~(size_t)0 ? ldg_stream16(p.kcache + oa + 32 * db + 8 * t) : make_uint4(0, 0, 0, 0);
            kb[db] = ob != ~(size_t)0 ? ldg_stream16(p.kcache + ob + 32 * db + 8 * t) : make_uint4(0, 0, 0, 0);
        }
    };

    float m_r[NT][2], l_r[NT][2];
    float o[D / 16][NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { m_r[nt][0] = -INFINITY; m_r[nt][1] = -INFINITY; l_r[nt][0] = 0.0f; l_r[nt][1] = 0.0f; }
#pragma unroll
    for (int dt = 0; dt < D / 16; ++dt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { o[dt][nt][0] = 0.0f; o[dt][nt][1] = 0.0f; o[dt][nt][2] = 0.0f; o[dt][nt][3] = 0.0f; }

    // ---- this warp's slices: warp, warp + 4, ... ---------------------------------------------------------------
    const int n_mine = nslices > warp ? (nslices - warp + WARPS - 1) / WARPS : 0;
    size_t off0 = slice_offsets(warp), off1 = slice_offsets(warp + WARPS);
    if (n_mine > 0) load_v(off0, warp, 0);
    cp_async_commit();
    if (n_mine > 1) load_v(off1, warp + WARPS, 1);
    cp_async_commit();
    uint4 ka[DB], kb[DB];
    if (n_mine > 0) load_k(off0, ka, kb);

    for (int i = 0; i < n_mine; ++i) {
        __syncwarp();                                        // everyone has finished reading the stage refilled below
        const size_t off2 = slice_offsets(warp + WARPS * (i + 2));
        if (i + 2 < n_mine) load_v(off2, warp + WARPS * (i + 2), (i + 2) % VSTAGES);
        cp_async_commit();

        // S^T = K Q^T : 16 keys x 8 rows per tile of rows
        const int k0 = kbegin + 16 * (warp + WARPS * i);
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { s[nt][0] = 0.0f; s[nt][1] = 0.0f; s[nt][2] = 0.0f; s[nt][3] = 0.0f; }
#pragma unroll
        for (int db = 0; db < DB; ++db) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const unsigned a1[4] = {ka[db].x, kb[db].x, ka[db].y, kb[db].y};
                const unsigned a2[4] = {ka[db].z, kb[db].z, ka[db].w, kb[db].w};
                mma_bf16(s[nt], a1, qf[nt][db].x, qf[nt][db].y);
                mma_bf16(s[nt], a2, qf[nt][db].z, qf[nt][db].w);
            }
        }
        if (i + 1 < n_mine) load_k(off1, ka, kb);            // next slice's keys: in flight during softmax and P V
        // visibility depends on the key only (one query position): keys k0 + g and k0 + g + 8
        const int ja = k0 + g, jb = ja + 8;
        const bool va = ja <= pos && ja >= lo && ja < kend, vb = jb <= pos && jb >= lo && jb < kend;
        unsigned pb0[NT], pb1[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float alpha[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {                    // c: row 2t + c of this tile
                const float sa = va ? s[nt][c] * p.scale_log2 : -INFINITY;
                const float sb = vb ? s[nt][2 + c] * p.scale_log2 : -INFINITY;
                float mx = fmaxf(sa, sb);
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_r[nt][c], mx);
                const float base = (m_new == -INFINITY) ? 0.0f : m_new;
                alpha[c] = exp2f(m_r[nt][c] - base);
                m_r[nt][c] = m_new;
                const float pa = exp2f(sa - base), pbv = exp2f(sb - base);
                s[nt][c] = pa;
                s[nt][2 + c] = pbv;
                l_r[nt][c] = l_r[nt][c] * alpha[c] + pa + pbv;   // this lane's keys only; summed over g at the end
            }
            if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {   // the maximum moved for some row
#pragma unroll
                for (int dt = 0; dt < D / 16; ++dt) {
                    o[dt][nt][0] *= alpha[0]; o[dt][nt][1] *= alpha[1];
                    o[dt][nt][2] *= alpha[0]; o[dt][nt][3] *= alpha[1];
                }
            }
            // P^T as B operand: transpose the two 8x8 blocks (keys 0-7 | 8-15) x (rows 0-7)
            pb0[nt] = movmatrix_trans(pack_bf16(s[nt][0], s[nt][1]));
            pb1[nt] = movmatrix_trans(pack_bf16(s[nt][2], s[nt][3]));
        }

        cp_async_wait<2>();                                  // V of slice i has landed (two younger groups may fly)
        __syncwarp();
        const bf16* vt = vs + (i % VSTAGES) * 16 * LDS;
#pragma unroll
        for (int dt = 0; dt < D / 16; ++dt) {
            unsigned a[4];
            ldmatrix_x4_trans(a, vt + ((lane & 7) + 8 * (lane >> 4)) * LDS + dt * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_bf16(o[dt][nt], a, pb0[nt], pb1[nt]);
        }
        off1 = off2;
    }
    cp_async_wait<0>();

    // ---- merge the four warps -----------------------------------------------------------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float v = l_r[nt][c];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            l_r[nt][c] = v;
        }
    __syncthreads();                                         // all warps are done with their V stages
    constexpr int ROWS = 8 * NT;
    float* mo = reinterpret_cast<float*>(smem_raw);          // [WARPS][ROWS][D]
    float* mm = mo + WARPS * ROWS * D;                       // [WARPS][ROWS]
    float* ml = mm + WARPS * ROWS;                           // [WARPS][ROWS]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int r = 8 * nt + 2 * t + c;
            float* dst = mo + (warp * ROWS + r) * D;
#pragma unroll
            for (int dt = 0; dt < D / 16; ++dt) {
                dst[dt * 16 + g] = o[dt][nt][c];
                dst[dt * 16 + g + 8] = o[dt][nt][2 + c];
            }
            if (g == 0) { mm[warp * ROWS + r] = m_r[nt][c]; ml[warp * ROWS + r] = l_r[nt][c]; }
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += 128) {
        const int r = idx / D, e = idx % D;
        float mstar = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mstar = fmaxf(mstar, mm[w * ROWS + r]);
        float lsum = 0.0f, acc = 0.0f;
        if (mstar != -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = exp2f(mm[w * ROWS + r] - mstar);
                lsum += ml[w * ROWS + r] * f;
                acc += mo[(w * ROWS + r) * D + e] * f;
            }
        }
        const size_t orow = (size_t)tok * p.nq + (size_t)(kvh * G + r);
        if (nsplits == 1) {
            p.out[orow * D + e] = __float2bfloat16_rn(lsum > 0.0f ? acc / lsum : 0.0f);
        } else {
            p.part_acc[(orow * p.max_splits + split) * D + e] = acc;
            if (e == 0) {
                p.part_ml[(orow * p.max_splits + split) * 2] = mstar;
                p.part_ml[(orow * p.max_splits + split) * 2 + 1] = lsum;
            }
        }
    }
}

template <int NT>
static size_t attn_decode_smem_bytes() {
    const size_t stages = (size_t)4 * 3 * 16 * (PI_HEAD_DIM + 8) * sizeof(bf16);
    const size_t merge = (size_t)4 * 8 * NT * (PI_HEAD_DIM + 2) * sizeof(float);
    return stages > merge ? stages : merge;
}

#if PI_HEAD_DIM % 32 == 0
template <int NT, bool CONTIG>
static int launch_attn_decode(const AttnParams& p, int num_segments, int splits, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = attn_decode_smem_bytes<NT>();
    auto kernel = attn_decode_kernel<PI_HEAD_DIM, NT, CONTIG>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "attention: cannot reserve %zu bytes of shared memory: %s", smem,
                     cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    pi_launch(kernel, dim3((unsigned)num_segments, p.nkv, splits), dim3(128), smem, stream, p);
    return pi_check_launch("pi_attention_mma decode");
}
#endif

// Combine the key ranges of decode-mode rows: one block per (token, head).
template <int D>
__global__ void attn_merge_kernel(const AttnParams p, const int* __restrict__ token_seg, const Prefetch pf) {
    if (pi_prefetch_role(pf)) return;
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;  // token * nq + head
    const int t = row / p.nq;
    const int seg = token_seg[t];
    if (p.seg_len[seg] != 1) return;
    const int n = decode_ranges(p.seg_start[seg], p.window, p.split_keys, p.max_splits);
    if (n <= 1) return;
    const float2* ml = reinterpret_cast<const float2*>(p.part_ml + (size_t)row * p.max_splits * 2);   // (max, sum)
    const float* acc = p.part_acc + (size_t)row * p.max_splits * D;
    // The ranges are taken eight at a time with all their loads issued before the first use: the loop is a chain
    // of memory latencies otherwise.  The order of the sums is the order of the ranges.
    float mstar = -INFINITY;
    for (int s0 = 0; s0 < n; s0 += 8) {
        float2 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = s0 + i < n ? ml[s0 + i] : make_float2(-INFINITY, 0.0f);
#pragma unroll
        for (int i = 0; i < 8; ++i) mstar = fmaxf(mstar, v[i].x);
    }
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float lsum = 0.0f, a = 0.0f;
        if (mstar != -INFINITY) {
            for (int s0 = 0; s0 < n; s0 += 8) {
                float2 v[8];
                float x[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool live = s0 + i < n;
                    v[i] = live ? ml[s0 + i] : make_float2(-INFINITY, 0.0f);
                    x[i] = live ? acc[(size_t)(s0 + i) * D + e] : 0.0f;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float f = exp2f(v[i].x - mstar);      // -inf gives 0
                    lsum += v[i].y * f;
                    a += x[i] * f;
                }
            }
        }
        p.out[(size_t)row * D + e] = __float2bfloat16_rn(lsum > 0.0f ? a / lsum : 0.0f);
    }
}

template <int ROW_WARPS, int KEY_WARPS, int STAGES>
static size_t attn_smem_bytes() {
    return (size_t)(ROW_WARPS * 16 + 2 * STAGES * BN) * (PI_HEAD_DIM + 8) * sizeof(bf16);
}

template <int ROW_WARPS, int KEY_WARPS, int STAGES>
static int launch_attn(const AttnParams& p, int num_segments, int splits, cudaStream_t stream) {
    static bool configured = false;  // once per process and kernel
    const size_t smem = attn_smem_bytes<ROW_WARPS, KEY_WARPS, STAGES>();
    auto kernel = attn_mma_kernel<PI_HEAD_DIM, ROW_WARPS, KEY_WARPS, STAGES>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "attention: cannot reserve %zu bytes of shared memory: %s", smem,
                     cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    const long long linear = (long long)num_segments * p.tiles_per_seg * p.nkv;
    if (KEY_WARPS == 1 && linear > 2147483647LL) return pi_refuse("pi_attention_mma: %lld tiles are beyond the grid limit", linear);
    const dim3 grid = KEY_WARPS == 1 ? dim3((unsigned)linear, 1, 1) : dim3((unsigned)num_segments * p.tiles_per_seg, p.nkv, splits);
    pi_launch(kernel, grid, dim3(ROW_WARPS * KEY_WARPS * 32), smem, stream, p);
    return pi_check_launch("pi_attention_mma");
}

PI_EXPORT int pi_attention_head_dim() { return PI_HEAD_DIM; }

// The number of key ranges a decoding request at position `pos` (0-based, its newest token) uses.
PI_EXPORT int pi_attention_num_splits(int pos, int window, int split_keys) {
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int lo_al = (lo / BN) * BN;
    return (pos + 1 - lo_al + split_keys - 1) / split_keys;
}

// has_prompt / has_decode say which kinds of segment the batch holds (a kernel is launched for each kind
// present); max_seg_len bounds the grid of the prompt kernel; max_splits is the width of the scratch and the
// grid depth of the decode kernel (>= the number of ranges of every decoding request in the batch).
// prefetch_ptr / prefetch_bytes: weights the next product will stream; the merge kernel's spare CTAs ask for them
// to be brought into L2 (null / 0: none).  has_decode = 2: the partial results of the key ranges are already in
// part_acc / part_ml (written by the tcgen05 decode kernel); only the merge runs.
PI_EXPORT int pi_attention_mma_prefetch(const void* q, int q_stride, const void* kcache, const void* vcache,
                               const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                               const int* seg_start, const int* seg_len, const int* token_seg, void* out,
                               float* part_acc, float* part_ml, int max_splits, int split_keys, int num_tokens,
                               int num_segments, int max_seg_len, int has_prompt, int has_decode, int nq, int nkv,
                               int page_size, int window, float scale, const void* prefetch_ptr,
                               unsigned long long prefetch_bytes, cudaStream_t stream) {
    if (num_tokens <= 0 || num_segments <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) return pi_refuse("pi_attention_mma: nq=%d must be a positive multiple of nkv=%d", nq, nkv);
    if (page_size <= 0) return pi_refuse("pi_attention_mma: page_size=%d must be positive", page_size);
    if (q_stride % 8 != 0) return pi_refuse("pi_attention_mma: q_stride=%d must be a multiple of 8 elements", q_stride);
    if (split_keys <= 0 || split_keys % BN != 0) return pi_refuse("pi_attention_mma: split_keys=%d must be a positive multiple of %d", split_keys, BN);
    if (nkv > 65535 || max_splits > 65535) return pi_refuse("pi_attention_mma: nkv=%d or max_splits=%d beyond the grid limit", nkv, max_splits);
    AttnParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride;
    p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.seg_off = seg_off; p.seg_slot = seg_slot; p.seg_start = seg_start; p.seg_len = seg_len;
    p.out = (bf16*)out; p.part_acc = part_acc; p.part_ml = part_ml; p.max_splits = max_splits;
    p.nq = nq; p.nkv = nkv; p.group = nq / nkv; p.page_size = page_size; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.split_keys = split_keys;
    p.num_segments = num_segments;
    int rc = 0;
    if (has_prompt) {
        p.decode = 0;
        const long long rows = (long long)max_seg_len * p.group;
        if (rows > 64) {   // long portions: 128 rows per CTA halve the key/value traffic per query
            p.tiles_per_seg = (int)((rows + 127) / 128);
            rc = launch_attn<8, 1, 2>(p, num_segments, 1, stream);
        } else {
            p.tiles_per_seg = (int)((rows + 63) / 64);
            rc = launch_attn<4, 1, 2>(p, num_segments, 1, stream);
        }
        if (rc) return rc;
    }
    if (has_decode) {
        if (max_splits < 1) return pi_refuse("pi_attention_mma: max_splits=%d must be at least 1", max_splits);
        if (max_splits > 1 && (part_acc == nullptr || part_ml == nullptr)) return pi_refuse("pi_attention_mma: scratch for %d key ranges is missing", max_splits);
        p.decode = 1;
        p.tiles_per_seg = (p.group + 15) / 16;
        if (has_decode == 2) {
            // the partial results were written by another kernel (same layout): only the merge runs here
        } else
#if PI_HEAD_DIM % 32 == 0
        if (p.group <= 8) rc = page_size % 16 == 0 ? launch_attn_decode<1, true>(p, num_segments, max_splits, stream)
                                                   : launch_attn_decode<1, false>(p, num_segments, max_splits, stream);
        else if (p.group <= 16) rc = page_size % 16 == 0 ? launch_attn_decode<2, true>(p, num_segments, max_splits, stream)
                                                         : launch_attn_decode<2, false>(p, num_segments, max_splits, stream);
        else rc = launch_attn<1, 4, 3>(p, num_segments, max_splits, stream);
#else
        rc = launch_attn<1, 4, 3>(p, num_segments, max_splits, stream);
#endif
        if (rc) return rc;
        if (max_splits > 1) {
            const Prefetch pf = pi_make_prefetch(prefetch_ptr, prefetch_bytes, num_tokens * nq);
            pi_launch(attn_merge_kernel<PI_HEAD_DIM>, dim3(num_tokens * nq + pi_prefetch_ctas(pf)), dim3(PI_HEAD_DIM >= 128 ? 128 : 64), 0, stream, p, token_seg, pf);
            rc = pi_check_launch("pi_attention_mma merge");
        }
    }
    return rc;
}

PI_EXPORT int pi_attention_mma(const void* q, int q_stride, const void* kcache, const void* vcache,
                               const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                               const int* seg_start, const int* seg_len, const int* token_seg, void* out,
                               float* part_acc, float* part_ml, int max_splits, int split_keys, int num_tokens,
                               int num_segments, int max_seg_len, int has_prompt, int has_decode, int nq, int nkv,
                               int page_size, int window, float scale, cudaStream_t stream) {
    return pi_attention_mma_prefetch(q, q_stride, kcache, vcache, block_table, bt_stride, seg_off, seg_slot, seg_start,
                                     seg_len, token_seg, out, part_acc, part_ml, max_splits, split_keys, num_tokens,
                                     num_segments, max_seg_len, has_prompt, has_decode, nq, nkv, page_size, window, scale,
                                     nullptr, 0, stream);
}

// ---------------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate (see attention_noalloc.h).
// The partial results of the split decode attention live in a fixed array in device memory that is
// part of this library's image: every GPU that loads the library holds PI_NOALLOC_SCRATCH_BYTES of it
// until the process exits.
// ---------------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_noalloc_scratch[PI_NOALLOC_SCRATCH_BYTES / sizeof(float)];

// Device addresses of g_noalloc_scratch, looked up once per device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use: the address comes from
// cudaGetSymbolAddress, asked while that device is current.
#define PI_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[PI_NOALLOC_MAX_DEVICES] = {nullptr};

static int noalloc_scratch(float** out) {
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        snprintf(g_pi_error, sizeof(g_pi_error), "pi_attention_mma_noalloc: cudaGetDevice: %s", cudaGetErrorString(err));
        return (int)err;
    }
    if (device < 0 || device >= PI_NOALLOC_MAX_DEVICES)
        return pi_refuse("pi_attention_mma_noalloc: device index %d is beyond the %d this library tracks", device, PI_NOALLOC_MAX_DEVICES);
    if (g_noalloc_ptr[device] == nullptr) {
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            snprintf(g_pi_error, sizeof(g_pi_error), "pi_attention_mma_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
            return err != cudaSuccess ? (int)err : -1;
        }
        g_noalloc_ptr[device] = (float*)ptr;
    }
    *out = g_noalloc_ptr[device];
    return 0;
}

PI_EXPORT int pi_attention_noalloc_scratch_bytes() { return PI_NOALLOC_SCRATCH_BYTES; }

PI_EXPORT int pi_attention_mma_noalloc(const void* q, int q_stride, const void* kcache, const void* vcache,
                                       const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                                       const int* seg_start, const int* seg_len, const int* token_seg, void* out,
                                       int max_splits, int split_keys, int num_tokens, int num_segments,
                                       int max_seg_len, int has_prompt, int has_decode, int nq, int nkv, int page_size,
                                       int window, float scale, cudaStream_t stream) {
    if (num_tokens <= 0 || num_segments <= 0) return 0;
    if (max_splits < 1) return pi_refuse("pi_attention_mma_noalloc: max_splits=%d must be at least 1", max_splits);
    if (nq <= 0 || nkv <= 0) return pi_refuse("pi_attention_mma_noalloc: nq=%d and nkv=%d must be positive", nq, nkv);
    // pi_attention_mma also knows has_decode = 2, "another kernel has already left the partial results in the
    // scratch, only merge them".  Nothing but this entry can write the fixed array, so here that would merge whatever
    // an earlier call left behind: refused.
    if (has_decode != 0 && has_decode != 1)
        return pi_refuse("pi_attention_mma_noalloc: has_decode=%d must be 0 or 1", has_decode);
    if (has_prompt != 0 && has_prompt != 1)
        return pi_refuse("pi_attention_mma_noalloc: has_prompt=%d must be 0 or 1", has_prompt);
    // partial outputs [tokens * heads, max_splits, D] followed by (max, sum) pairs [tokens * heads, max_splits, 2]
    const unsigned long long rows = (unsigned long long)num_tokens * (unsigned long long)(nq > 0 ? nq : 0);
    const unsigned long long acc_floats = rows * (unsigned long long)max_splits * PI_HEAD_DIM;
    const unsigned long long need = (acc_floats + rows * (unsigned long long)max_splits * 2ull) * sizeof(float);
    if (need > (unsigned long long)PI_NOALLOC_SCRATCH_BYTES)
        return pi_refuse("pi_attention_mma_noalloc: %d tokens x %d heads x %d key ranges need %llu bytes of scratch, the fixed "
                         "array holds %d; use pi_attention_mma with scratch of your own", num_tokens, nq, max_splits, need,
                         PI_NOALLOC_SCRATCH_BYTES);
    float* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    // Nothing in the scratch has to start at zero: a (row, range) entry is written by the attention kernel
    // before the merge kernel reads it, and entries of ranges a request does not use are never read.
    return pi_attention_mma(q, q_stride, kcache, vcache, block_table, bt_stride, seg_off, seg_slot, seg_start, seg_len,
                            token_seg, out, scratch, scratch + acc_floats, max_splits, split_keys, num_tokens,
                            num_segments, max_seg_len, has_prompt, has_decode, nq, nkv, page_size, window, scale, stream);
}

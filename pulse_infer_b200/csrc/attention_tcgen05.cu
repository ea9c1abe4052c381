// Paged flash attention for prompt portions on the 5th-generation tensor cores (bfloat16).
//
// A CTA owns 256 query rows - (token, head-in-group) pairs of one kv head of one request segment, as in
// attention_mma.cu - as two query tiles of 128, and walks the visible keys in tiles of 128:
//   S_x = Q_x K^T   tcgen05.mma, M 128 x N 128, both operands K-major from 128-byte-swizzled shared memory,
//                   accumulator in tensor memory (128 columns per query tile)
//   softmax         four warps per query tile, ONE THREAD PER ROW: the row's scores come out of tensor memory
//                   with tcgen05.ld, so max / exp2 / sum need no shuffles.  The probabilities go back into
//                   tensor memory as bf16 pairs over the scores already read (tcgen05.st).  The reference
//                   point of the exponentials moves only when the maximum grew by more than 2^8, so the
//                   running output is rescaled (tcgen05.ld / st) rarely.
//   O_x += P_x V    tcgen05.mma with the A operand from tensor memory and V from shared memory, MN-major
//                   (rows of V are keys)
// While one query tile is in its softmax the tensor pipe works for the other.  Tensor memory: S_0, S_1, O_0,
// O_1 of 128 columns each - all 512.  Keys and values arrive by TMA through a ring of tiles (K(0) V(0) K(1)
// ...), one box per (page, 64-wide half of the head): cp.async.bulk.tensor.2d over the page pool seen as a
// [pages * kv heads * page size, head size] matrix; the lanes of the producer warp look the page ids up in
// the block table together.  Roles: warp 0 TMA producer, warp 1 MMA issuer + owner of tensor memory, warps
// 2-5 softmax / output of query tile 0, warps 6-9 of query tile 1.
// Every mbarrier wait is bounded; on a timeout the kernel records a code, all roles fall through and tensor
// memory is freed.
//
// Needs: head size 64 or 128 (PI_HEAD_DIM), page size in {8, 16, 32, 64, 128}.  Segments of one token are
// left to the decode kernel.
//
// Reference parity: src/ops/kernels/cuda/paged_attention.cu:65-137 (grouping, 1/sqrt(d) scale, causal bound
// by absolute position, online softmax, out = acc / sum).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "common.cuh"

#ifndef PI_HEAD_DIM
#error "compile with -DPI_HEAD_DIM=64 or 128"
#endif

#if PI_HEAD_DIM == 64 || PI_HEAD_DIM == 128

#define FA_BM 128            // rows of a query tile
#define FA_ROWS 256          // rows of a CTA: two query tiles
#define FA_BN 128            // keys of a tile
#define FA_STAGES 5          // ring of K / V tiles
#define FA_THREADS 320
#define FA_SPIN_LIMIT (1u << 22)

__device__ unsigned g_fa_status;

struct FaParams {
    const bf16* q; int q_stride;
    const int* block_table; int bt_stride;
    const int* seg_off; const int* seg_slot; const int* seg_start; const int* seg_len;
    bf16* out;
    int nq, nkv, group;
    int page_size, window;
    float scale_log2;
    int tiles_per_seg, num_segments;
    // key splitting for short portions behind long contexts: gridDim.y CTAs share the key tiles of a query block and
    // leave (reference point of the exponentials, sum, unnormalised output) per row for attn_prompt_merge_kernel
    int splits;
    float* part_acc;       // [tokens * nq][splits][D]
    float* part_ml;        // [tokens * nq][splits][2]
};

// ---- PTX wrappers (see gemm_tcgen05.cu for the same set with comments) ------------------------------------
__device__ __forceinline__ unsigned fa_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem(bar)), "r"(count));
}
__device__ __forceinline__ void fa_mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fa_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fa_mbar_wait(void* bar, unsigned parity, unsigned code, volatile unsigned* failed) {
    for (unsigned spin = 0; spin < FA_SPIN_LIMIT; ++spin) {
        unsigned ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(fa_smem(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    atomicCAS(&g_fa_status, 0u, code);
    return false;
}
__device__ __forceinline__ void fa_tma_load(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(fa_smem(dst)), "l"(map), "r"(fa_smem(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fa_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// A operand from tensor memory (rows = lanes, two bf16 per 32-bit column), B from shared memory
__device__ __forceinline__ void fa_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_commit(void* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ void fa_tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fa_tmem_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void fa_tmem_st16(unsigned taddr, const unsigned (&w)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "r"(w[8]), "r"(w[9]),
          "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15])
        : "memory");
}

// K-major operand tile: rows of 128 bytes (64 bf16), 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long fa_desc_kmajor(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand (V as the B operand of P V: its rows are keys = the k index, the head dimension is
// contiguous): 128-byte swizzle, blocks of 64 elements along the head dimension `lbo` bytes apart,
// groups of 8 keys 1024 bytes apart
__device__ __forceinline__ unsigned long long fa_desc_mnmajor(unsigned addr, unsigned lbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}

__device__ __forceinline__ float fa_ex2(float x) {   // 2^x; -inf gives 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ int fa_window_lo(int pos, int window) {
    return (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
}

// One pass of a row over a 128-key tile of scores in TMEM.  MASKED: keys outside [lo_r, pos_r] or at / beyond
// kend count as -inf.  Pass 1 returns the row's maximum of the raw scores.
template <bool MASKED>
__device__ __forceinline__ float fa_row_max(unsigned tmem_row, int k0, int pos_r, int lo_r, int kend) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < FA_BN; c += 32) {
        float v[32];
        fa_tmem_ld32(tmem_row + c, v);
        if (MASKED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int key = k0 + c + i;
                if (!(key <= pos_r && key >= lo_r && key < kend)) v[i] = -INFINITY;
            }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, v[i]); m1 = fmaxf(m1, v[i + 1]); m2 = fmaxf(m2, v[i + 2]); m3 = fmaxf(m3, v[i + 3]);
        }
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// Pass 2: p = 2^(s * scale - base) as bf16, two to a 32-bit column, written over the row's own scores (the 32
// scores of a chunk are read before the 16 columns that replace scores already read are written); returns
// the row's sum.
template <bool MASKED>
__device__ __forceinline__ float fa_row_probs(unsigned tmem_row, float scale_log2, float base, int k0, int pos_r, int lo_r, int kend) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    const float nbase = -base;
#pragma unroll 1
    for (int c = 0; c < FA_BN; c += 32) {
        float v[32];
        fa_tmem_ld32(tmem_row + c, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float pv = fa_ex2(fmaf(v[i], scale_log2, nbase));
            if (MASKED) {
                const int key = k0 + c + i;
                if (!(key <= pos_r && key >= lo_r && key < kend)) pv = 0.0f;
            }
            v[i] = pv;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) { s0 += v[i]; s1 += v[i + 1]; s2 += v[i + 2]; s3 += v[i + 3]; }
        unsigned w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);     // the even key in the low half
            w[i] = *reinterpret_cast<unsigned*>(&t);
        }
        fa_tmem_st16(tmem_row + c / 2, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    return (s0 + s1) + (s2 + s3);
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
attn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const FaParams p) {
    constexpr int HALVES = D / 64;                       // 64-wide (128-byte) column blocks of the head
    constexpr unsigned HALF_BYTES = 128 * 128;           // 128 rows x 128 bytes
    constexpr unsigned TILE_BYTES = HALVES * HALF_BYTES; // a Q, K or V tile: 128 rows x D bf16
    constexpr unsigned TMEM_COLS = 512;
    constexpr unsigned S_COL = 0, O_COL = 256;           // S of query tile x at S_COL + 128 x (P over its first 64 columns), O at O_COL + 128 x

    // ---- which rows -------------------------------------------------------------------------------------
    const int kvh = blockIdx.x % p.nkv;
    const int rest = blockIdx.x / p.nkv;
    const int tile = p.tiles_per_seg - 1 - rest / p.num_segments;     // tiles with the most keys first
    const int seg = rest % p.num_segments;
    const int len = p.seg_len[seg];
    if (len == 1) return;                                 // single tokens go to the decode kernel
    const int G = p.group;
    const int rows_total = len * G;
    const int row0 = tile * FA_ROWS;
    if (row0 >= rows_total) return;
    const bool two = row0 + FA_BM < rows_total;           // the second query tile has rows
    const int start = p.seg_start[seg], tok_off = p.seg_off[seg];
    const int* table = p.block_table + (size_t)p.seg_slot[seg] * p.bt_stride;
    const int row_last = min(row0 + FA_ROWS, rows_total) - 1;
    const int pos_first = start + row0 / G, pos_last = start + row_last / G;
    int kbegin = (fa_window_lo(pos_first, p.window) / FA_BN) * FA_BN;
    const int kend = pos_last + 1;
    int num_tiles = (kend - kbegin + FA_BN - 1) / FA_BN;
    const int split = blockIdx.y;
    if (p.splits > 1) {
        // this CTA's share of the key tiles (contiguous, as even as it goes); a share may be empty
        const int t0 = (int)((long long)split * num_tiles / p.splits), t1 = (int)((long long)(split + 1) * num_tiles / p.splits);
        kbegin += t0 * FA_BN;
        num_tiles = t1 - t0;
        if (num_tiles <= 0) {
            pdl_wait();
            for (int r = threadIdx.x; r < FA_ROWS; r += FA_THREADS) {
                const int rf = row0 + r;
                if (rf < rows_total) {
                    const size_t orow = (size_t)(tok_off + rf / G) * p.nq + kvh * G + rf % G;
                    p.part_ml[(orow * p.splits + split) * 2] = -INFINITY;
                    p.part_ml[(orow * p.splits + split) * 2 + 1] = 0.0f;
                }
            }
            return;
        }
    }

    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;                             // [2 query tiles][HALVES][128 rows][128 B]
    unsigned char* sKV = sQ + 2 * TILE_BYTES;             // [FA_STAGES][HALVES][128 keys][128 B]: K0 V0 K1 V1 ... in a ring
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sKV + FA_STAGES * TILE_BYTES);
    unsigned long long* full = bars;                      // [FA_STAGES] TMA -> MMA: the tile of a stage has landed
    unsigned long long* empty = bars + FA_STAGES;         // [FA_STAGES] MMA -> TMA: the products that read it are done
    unsigned long long* s_full = bars + 2 * FA_STAGES;    // [2] MMA -> softmax of query tile x: scores are in TMEM
    unsigned long long* p_ready = s_full + 2;             // [2] softmax (4 warps) -> MMA: P written, O rescaled, S read
    unsigned long long* pv_done = s_full + 4;             // [2] MMA -> softmax: O updated, P free
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(s_full + 6);
    volatile unsigned* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < FA_STAGES; ++i) { fa_mbar_init(&full[i], 1); fa_mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { fa_mbar_init(&s_full[i], 1); fa_mbar_init(&p_ready[i], 4); fa_mbar_init(&pv_done[i], 1); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_smem(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the ring starts as zeros: rows of a value tile that no page fills must not hold NaN bit patterns (0 x NaN)
    for (unsigned i = threadIdx.x; i < FA_STAGES * TILE_BYTES / 16; i += FA_THREADS) reinterpret_cast<uint4*>(sKV)[i] = make_uint4(0, 0, 0, 0);
    pdl_wait();   // q and the pages are written by the kernels before this one; all above touched this CTA only
    // Q: thread r of the softmax warps copies row r into the swizzled K-major layout (16-byte chunk c of a
    // 128-byte row goes to chunk c ^ (row & 7))
    if (warp >= 2) {
        const int r = (warp - 2) * 32 + lane;             // 0..255
        const int rf = row0 + r;
        const bool valid = rf < rows_total;
        const bf16* src = p.q + (size_t)(tok_off + (valid ? rf / G : 0)) * p.q_stride + (size_t)(kvh * G + (valid ? rf % G : 0)) * D;
        unsigned char* dst = sQ + (r >> 7) * TILE_BYTES + (r & 127) * 128;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            const uint4 v = valid ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0, 0, 0, 0);
            const int half = c / 8, cc = c % 8;
            *reinterpret_cast<uint4*>(dst + half * HALF_BYTES + ((cc ^ (r & 7)) << 4)) = v;
        }
    }
    fa_fence_async_smem();        // generic-proxy writes above become visible to TMA / tcgen05.mma
    fa_fence_before();
    __syncthreads();
    fa_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer: lane = page of the key tile ----------------
        // Loads run K(0) V(0) K(1) V(1) ... through the ring.  The lanes look their pages up in the block
        // table together (the lookups are the long latency here) and each issues the boxes of its own page.
        const int ps = p.page_size, pages_per_tile = FA_BN / ps;
        const unsigned page_bytes = (unsigned)ps * 128u;            // one (page, half) box
        auto lookup = [&](int j) -> int {
            const int key = kbegin + j * FA_BN + lane * ps;
            return (j < num_tiles && lane < pages_per_tile && key < kend) ? table[key / ps] : -1;
        };
        int page = lookup(0);
        for (int j = 0; j < num_tiles && !*failed; ++j) {
            const int next_page = lookup(j + 1);
            const unsigned mask = __ballot_sync(0xffffffffu, page >= 0);
            const unsigned bytes = (unsigned)__popc(mask) * page_bytes * HALVES;
            const int row = (page * p.nkv + kvh) * ps;
            bool ok = true;
#pragma unroll
            for (int isv = 0; isv < 2; ++isv) {
                const int n = 2 * j + isv, st = n % FA_STAGES, use = n / FA_STAGES;
                if (use > 0 && !fa_mbar_wait(&empty[st], (use - 1) & 1, (1u << 24) | n, failed)) { ok = false; break; }
                if (lane == 0) fa_mbar_expect_tx(&full[st], bytes);
                __syncwarp();
                if (page >= 0) {
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        fa_tma_load(sKV + st * TILE_BYTES + h * HALF_BYTES + lane * page_bytes, isv ? &map_v : &map_k, h * 64, row, &full[st]);
                }
            }
            if (!ok) break;
            page = next_page;
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // bf16 x bf16 -> f32, M 128; S: N 128, both K-major; PV: N D, B MN-major
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FA_BN >> 3) << 17) | ((unsigned)(FA_BM >> 4) << 24);
            const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) | ((unsigned)(FA_BM >> 4) << 24);
            const int nx = two ? 2 : 1;
            auto wait_full = [&](int n) -> bool { return fa_mbar_wait(&full[n % FA_STAGES], (n / FA_STAGES) & 1, (2u << 24) | n, failed); };
            auto issue_s = [&](int x, int j) {     // S_x(j) = Q_x K(j)^T
                const unsigned char* kt = sKV + ((2 * j) % FA_STAGES) * TILE_BYTES;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        fa_mma(tmem_base + S_COL + x * 128, fa_desc_kmajor(fa_smem(sQ + x * TILE_BYTES + h * HALF_BYTES) + k * 32),
                               fa_desc_kmajor(fa_smem(kt + h * HALF_BYTES) + k * 32), idesc_s, (h > 0 || k > 0) ? 1u : 0u);
                fa_commit(&s_full[x]);
            };
            bool ok = wait_full(0);
            if (ok) {
                fa_fence_after();
                for (int x = 0; x < nx; ++x) issue_s(x, 0);
                fa_commit(&empty[0]);                                  // K(0) is no longer read
            }
            for (int j = 0; j < num_tiles && ok && !*failed; ++j) {
                const bool have_next = j + 1 < num_tiles;
                if (!wait_full(2 * j + 1)) break;                      // V(j)
                if (have_next && !wait_full(2 * j + 2)) break;         // K(j + 1)
                const unsigned char* vt = sKV + ((2 * j + 1) % FA_STAGES) * TILE_BYTES;
                for (int x = 0; x < nx; ++x) {
                    if (!fa_mbar_wait(&p_ready[x], j & 1, (4u << 24) | (x << 20) | j, failed)) { ok = false; break; }
                    fa_fence_after();
                    // O_x += P_x V: 8 steps of 16 keys, P from tensor memory (8 columns a step); then the next
                    // scores of this query tile, which overwrite P_x: the tensor pipe runs its products in order
#pragma unroll
                    for (int kk = 0; kk < FA_BN / 16; ++kk)
                        fa_mma_ts(tmem_base + O_COL + x * 128, tmem_base + S_COL + x * 128 + kk * 8,
                                  fa_desc_mnmajor(fa_smem(vt) + kk * 16 * 128, HALF_BYTES), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    fa_commit(&pv_done[x]);
                    if (have_next) issue_s(x, j + 1);
                }
                if (!ok) break;
                fa_commit(&empty[(2 * j + 1) % FA_STAGES]);            // V(j) is no longer read
                if (have_next) fa_commit(&empty[(2 * j + 2) % FA_STAGES]);   // nor is K(j + 1)
            }
        }
    } else {
        // ---------------- softmax and output: thread = row; warps 2-5 query tile 0, warps 6-9 query tile 1 ----------------
        const int x = (warp - 2) >> 2;
        const int quarter = warp & 3;                      // TMEM lanes 32 * quarter .. + 31
        const int r = quarter * 32 + lane;                 // row in the query tile
        const int rf = row0 + x * FA_BM + r;
        if (x == 0 || two) {
            const bool row_valid = rf < rows_total;
            const int pos_r = row_valid ? start + rf / G : -1;
            const int lo_r = row_valid ? fa_window_lo(pos_r, p.window) : 0;
            const unsigned lane_base = (unsigned)(quarter * 32) << 16;
            const unsigned tmem_s = tmem_base + S_COL + x * 128 + lane_base;
            const unsigned tmem_o = tmem_base + O_COL + x * 128 + lane_base;
            // the rows of this query tile: a key tile is taken without masks when all of them see all of it
            const int xrow0 = row0 + x * FA_BM;
            const bool rows_full = xrow0 + FA_BM <= rows_total;
            const int xpos_first = start + xrow0 / G;
            const int xlo_last = fa_window_lo(start + (min(xrow0 + FA_BM, rows_total) - 1) / G, p.window);
            float m_run = -INFINITY, l_run = 0.0f;
            bool alive = true;
            for (int j = 0; j < num_tiles && alive; ++j) {
                const int k0 = kbegin + j * FA_BN;
                if (!fa_mbar_wait(&s_full[x], j & 1, (5u << 24) | (x << 20) | j, failed)) { alive = false; break; }
                fa_fence_after();
                const bool full_tile = rows_full && k0 + FA_BN - 1 <= xpos_first && k0 >= xlo_last && k0 + FA_BN <= kend;
                const float mx = (full_tile ? fa_row_max<false>(tmem_s, k0, pos_r, lo_r, kend)
                                            : fa_row_max<true>(tmem_s, k0, pos_r, lo_r, kend)) * p.scale_log2;   // the scale is positive
                // The reference point of the exponentials moves only when the maximum grew by more than 2^8:
                // probabilities stay below 256, and the running output is rescaled rarely.
                float alpha = 1.0f;
                if (mx > m_run + 8.0f) { alpha = fa_ex2(m_run - mx); m_run = mx; }     // m_run = -inf gives alpha 0
                const float base = (m_run == -INFINITY) ? 0.0f : m_run;
                // the previous P V of this query tile must be complete before O is rescaled and P is overwritten
                if (j > 0 && !fa_mbar_wait(&pv_done[x], (j - 1) & 1, (6u << 24) | (x << 20) | j, failed)) { alive = false; break; }
                fa_fence_after();
                if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        float o[32];
                        fa_tmem_ld32(tmem_o + c, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= alpha;
                        fa_tmem_st32(tmem_o + c, o);
                    }
                }
                const float lsum = full_tile ? fa_row_probs<false>(tmem_s, p.scale_log2, base, k0, pos_r, lo_r, kend)
                                             : fa_row_probs<true>(tmem_s, p.scale_log2, base, k0, pos_r, lo_r, kend);
                l_run = l_run * alpha + lsum;
                fa_fence_before();
                __syncwarp();
                if (lane == 0) fa_mbar_arrive(&p_ready[x]);
            }
            // ---------------- output: O / l ----------------
            if (alive && num_tiles > 0 && fa_mbar_wait(&pv_done[x], (num_tiles - 1) & 1, (7u << 24) | (x << 20), failed)) {
                fa_fence_after();
                if (p.splits > 1) {
                    // a share of the keys: the merge kernel divides by the sum of all shares
                    const size_t orow_i = row_valid ? (size_t)(tok_off + rf / G) * p.nq + kvh * G + rf % G : 0;
                    if (row_valid) {
                        p.part_ml[(orow_i * p.splits + split) * 2] = l_run > 0.0f ? m_run : -INFINITY;
                        p.part_ml[(orow_i * p.splits + split) * 2 + 1] = l_run;
                    }
                    float* acc = p.part_acc + (orow_i * p.splits + split) * D;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        float o[32];
                        fa_tmem_ld32(tmem_o + c, o);           // the whole warp loads; only rows that exist store
                        if (row_valid) {
#pragma unroll
                            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(acc + c + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                        }
                    }
                } else {
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                bf16* orow = p.out + (size_t)(tok_off + (row_valid ? rf / G : 0)) * p.nq * D + (size_t)(kvh * G + (row_valid ? rf % G : 0)) * D;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    float o[32];
                    fa_tmem_ld32(tmem_o + c, o);
                    if (row_valid) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 w;
                            __nv_bfloat162 t0 = __floats2bfloat162_rn(o[q4 * 8 + 0] * inv, o[q4 * 8 + 1] * inv);
                            __nv_bfloat162 t1 = __floats2bfloat162_rn(o[q4 * 8 + 2] * inv, o[q4 * 8 + 3] * inv);
                            __nv_bfloat162 t2 = __floats2bfloat162_rn(o[q4 * 8 + 4] * inv, o[q4 * 8 + 5] * inv);
                            __nv_bfloat162 t3 = __floats2bfloat162_rn(o[q4 * 8 + 6] * inv, o[q4 * 8 + 7] * inv);
                            w.x = *reinterpret_cast<unsigned*>(&t0); w.y = *reinterpret_cast<unsigned*>(&t1);
                            w.z = *reinterpret_cast<unsigned*>(&t2); w.w = *reinterpret_cast<unsigned*>(&t3);
                            *reinterpret_cast<uint4*>(orow + c + q4 * 8) = w;
                        }
                    }
                }
                }
            }
        }
    }
    // ---------------- common exit ----------------
    fa_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        fa_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Combine the shares of the keys that attn_tcgen05_kernel left for the rows of prompt portions: one block per
// (token, head), one thread per element of the head.  out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s, the shares
// taken in order; a share that saw no key (l = 0) is skipped.
template <int D>
__global__ void attn_prompt_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits,
                                         bf16* __restrict__ out, const int* __restrict__ token_seg,
                                         const int* __restrict__ seg_len, int nq) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x, t = row / nq;
    if (seg_len[token_seg[t]] == 1) return;          // single tokens are the decode kernel's
    const float2* ml = reinterpret_cast<const float2*>(part_ml + (size_t)row * splits * 2);
    const float* acc = part_acc + (size_t)row * splits * D;
    float mstar = -INFINITY;
    for (int s = 0; s < splits; ++s) {
        const float2 v = ml[s];
        if (v.y > 0.0f) mstar = fmaxf(mstar, v.x);
    }
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float num = 0.0f, den = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float2 v = ml[s];
            if (v.y > 0.0f) {
                const float w = fa_ex2(v.x - mstar);
                num += w * acc[(size_t)s * D + e];
                den += w * v.y;
            }
        }
        out[(size_t)row * D + e] = __float2bfloat16_rn(den > 0.0f ? num / den : 0.0f);
    }
}

// =============================================================================================================
// Decode: segments of one token.  The work is all memory traffic - every key and value of the request is read
// once for a handful of query rows - so the kernel is built around keeping HBM busy: one persistent CTA per SM,
// whose TMA producer warp runs ahead through a ring of key/value tiles ACROSS the boundaries of its pieces of
// work, so the ring never drains while a piece finishes.
//   S^T = K Q^T     tcgen05.mma M 128 (keys of the tile) x N 16 (the group's query heads, padded): the key tile
//                   that TMA delivered is the A operand as it lies; the scores land in tensor memory with one
//                   key per lane
//   softmax         four warps, thread = key: column maxima by warp shuffles and one exchange through shared
//                   memory per tile; every thread keeps the running maxima (the same in all threads) and the
//                   sum over ITS keys, which is reduced across threads once per piece
//   O^T += V^T P^T  tcgen05.mma M 128 (head dimension) x N 16, A = the value tile MN-major, B = the
//                   probabilities [16 heads, 128 keys] from shared memory
// Work split.  The key tiles (128 keys) of all (request, kv head) pairs of the step form one sequence - request after
// request, kv head after kv head, oldest tile first, each pair preceded by `pair_cost` units that stand for the fixed
// cost of starting and finishing it - and every CTA takes an equal span of it, whatever the lengths of the requests
// are: a span may end in the middle of a pair and the next CTA goes on from there.  A pair that lies inside one span
// is finished by its CTA.  A pair that was cut leaves (max, sum, accumulator) per piece in a scratch that is indexed
// by CTA (a span has at most one piece that began before it and one that goes on behind it, so two slots per CTA do
// for any batch and any context); when a CTA has done its span it reports its pieces, and the CTA that reports the
// pair's last missing piece - a counter per pair tells - adds the pieces up in the order of the keys and writes the
// output.  Nothing waits for another CTA.  The cuts depend on the whole step, so a request's result depends on its
// neighbours by rounding.
// Warps: 0 TMA producer, 1 MMA issuer, 2-5 softmax and output, 6 (fused mode) the writer of the new tokens' keys and
// values, which runs ahead of the producer.
// Needs a group of at most 16 query heads per kv head, pages of at most 64 keys, at most FD_MAX_SEGS segments.
// =============================================================================================================
#define FD_THREADS 224
#define FD_STAGES (PI_HEAD_DIM == 128 ? 3 : 6)
#define FD_MAX_SEGS 1024

struct FdParams {
    const bf16* q; int q_stride;
    const int* block_table; int bt_stride;
    const int* seg_off; const int* seg_slot; const int* seg_start; const int* seg_len;
    bf16* out;
    float* ws_acc;            // [CTAs][2 slots][16 heads][D]   accumulators of pieces of cut pairs
    float* ws_ml;             // [CTAs][2 slots][16 heads][2]   their (max, sum)
    unsigned* ws_count;       // [CTAs] pieces delivered of the pair that BEGINS in that CTA's span; zero between launches
    int span_min;             // shortest span in units
    int pair_cost;            // units a pair counts for beside its tiles
    // fuse = 1: q holds the raw q/k/v projections of the step's tokens [T, (nq + 2 nkv) D].  The kernel then does what
    // qk_norm_rope_write_kernel (elementwise.cu) does for single tokens: the queries of a piece are normalised per head
    // and rotated as they are loaded; the piece that holds a request's newest position normalises and rotates that
    // token's key, writes it and the value into their page, and only then requests the tile that contains it.
    int fuse;
    bf16* kpool; bf16* vpool;            // [pages][nkv][page_size][D]
    const void* qw; const void* kw;      // per-head norm weights [D] (bf16, or float if w_f32); null: no norm
    int w_f32; float eps;
    const float* cos_t; const float* sin_t; int rot_pairs;   // [T][rot_pairs]; adjacent pairs (2i, 2i + 1); null: no rotation
    int* error_count;                    // tokens whose page is missing are counted here, not written
    int nq, nkv, group;
    int page_size, window;
    float scale_log2;
    int num_segments;
};

// a piece: tiles [j0, j0 + ntiles) of the pair (seg, kvh)
struct FdItem {
    int seg, kvh, pos, lo, kb, ke, ntiles;
    int whole;        // the piece is the whole pair: its CTA writes the output
    int newest;       // the piece holds the pair's last tile (with the newest key)
    int slot;         // scratch slot of a piece of a cut pair: 1 if the pair begins in this span, else 0
    int cta_first;    // CTA whose span holds the pair's first tile
    int pieces;       // spans the pair reaches into
};

// key tiles of a segment's pairs: from the window's first key (rounded down to 64) to the newest one; 0 if the
// segment is not a single token
__device__ __forceinline__ int fd_seg_tiles(const FdParams& p, int seg) {
    if (p.seg_len[seg] != 1) return 0;
    const int pos = p.seg_start[seg];
    const int lo_al = (fa_window_lo(pos, p.window) / 64) * 64;
    return (pos + 1 - lo_al + FA_BN - 1) / FA_BN;
}

struct FdCursor { int f, end, seg, span; };

// tile_pre[s] = tiles per kv head of the segments before s, dec_pre[s] = single-token segments before s (shared
// memory); the sequence's first unit of segment s
__device__ __forceinline__ int fd_seg_unit(const FdParams& p, const int* tile_pre, int s) {
    return p.nkv * (tile_pre[s] + p.pair_cost * tile_pre[FD_MAX_SEGS + 1 + s]);
}

// the CTA's span
__device__ __forceinline__ void fd_begin(const FdParams& p, const int* tile_pre, FdCursor& c) {
    const int total = fd_seg_unit(p, tile_pre, p.num_segments);
    c.span = max((total + (int)gridDim.x - 1) / (int)gridDim.x, p.span_min);
    const long long b = (long long)blockIdx.x * c.span;
    c.f = (int)(b < total ? b : total);
    c.end = min(c.f + c.span, total);
    // the last segment whose first unit is not behind f
    int lo = 0, hi = p.num_segments;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (fd_seg_unit(p, tile_pre, mid) <= c.f) lo = mid; else hi = mid;
    }
    c.seg = lo;
}

// the next piece of this CTA's span
__device__ __forceinline__ bool fd_next(const FdParams& p, const int* tile_pre, FdCursor& c, FdItem& w) {
    while (c.f < c.end) {
        while (fd_seg_unit(p, tile_pre, c.seg + 1) <= c.f) ++c.seg;      // ends: f is before the end of the sequence
        const int n = tile_pre[c.seg + 1] - tile_pre[c.seg];
        const int per = n + p.pair_cost;
        const int rel = c.f - fd_seg_unit(p, tile_pre, c.seg);
        const int tile0 = c.f - rel % per + p.pair_cost;                  // unit of the pair's first tile
        const int lo_u = max(c.f, tile0), hi_u = min(c.end, tile0 + n);
        if (hi_u <= lo_u) {          // the span ends among the pair's cost units: its tiles are the next CTA's
            c.f = c.end;
            break;
        }
        const int j0 = lo_u - tile0;
        w.seg = c.seg;
        w.kvh = rel / per;
        w.ntiles = hi_u - lo_u;
        w.pos = p.seg_start[w.seg];
        w.lo = fa_window_lo(w.pos, p.window);
        w.kb = (w.lo / 64) * 64 + j0 * FA_BN;
        w.newest = (j0 + w.ntiles == n) ? 1 : 0;
        w.ke = w.newest ? w.pos + 1 : w.kb + w.ntiles * FA_BN;
        w.whole = (j0 == 0 && w.newest) ? 1 : 0;
        w.slot = j0 == 0 ? 1 : 0;
        w.cta_first = tile0 / c.span;
        w.pieces = (tile0 + n - 1) / c.span - w.cta_first + 1;
        c.f = hi_u;
        return true;
    }
    return false;
}

// GP (4, 8 or 16) columns of a row of tensor memory
template <int GP>
__device__ __forceinline__ void fa_tmem_ld_cols(unsigned taddr, float (&v)[GP]) {
    unsigned r[16];
    if constexpr (GP == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    } else if constexpr (GP == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr) : "memory");
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < GP; ++i) v[i] = __uint_as_float(r[i]);
}
template <int GP>
__device__ __forceinline__ void fa_tmem_st_cols(unsigned taddr, const float (&v)[GP]) {
    if constexpr (GP == 4) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                     ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])) : "memory");
    } else if constexpr (GP == 8) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                       "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])) : "memory");
    } else {
        unsigned w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(v[i]);
        fa_tmem_st16(taddr, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fa_warp_max(float v) {      // one instruction on sm_100a
    float m;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(m) : "f"(v));
    return m;
}
__device__ __forceinline__ void fd_softmax_sync() {       // the four softmax warps
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// a counter in shared memory that another warp of the CTA raises: bounded like the waits on barriers
__device__ __forceinline__ void fd_set_count(int* counter, int value) {
    asm volatile("st.release.cta.shared::cta.b32 [%0], %1;" ::"r"(fa_smem(counter)), "r"(value) : "memory");
}
__device__ __forceinline__ bool fd_wait_count(int* counter, int want, unsigned code, volatile unsigned* failed) {
    for (unsigned spin = 0; spin < FA_SPIN_LIMIT; ++spin) {
        int have;
        asm volatile("ld.acquire.cta.shared::cta.b32 %0, [%1];" : "=r"(have) : "r"(fa_smem(counter)) : "memory");
        if (have >= want) return true;
        if ((spin & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    atomicCAS(&g_fa_status, 0u, code);
    return false;
}

__device__ __forceinline__ float fd_weight(const void* w, int w_f32, int i) {
    return w_f32 ? reinterpret_cast<const float*>(w)[i] : __bfloat162float(reinterpret_cast<const bf16*>(w)[i]);
}

// The newest token of item w's request: its key (normalised, rotated) and value go into their page.  One warp; lane
// takes four elements (two adjacent pairs), the arithmetic of qk_norm_rope_write_kernel in the same order.
template <int D>
__device__ __forceinline__ void fd_write_new_token(const FdParams& p, const FdItem& w, const int* table, int lane) {
    const int tok = p.seg_off[w.seg];
    const int page = table[w.pos / p.page_size];
    if (page < 0) {
        if (lane == 0) atomicAdd(p.error_count, 1);
        return;
    }
    const size_t dst = (((size_t)page * p.nkv + w.kvh) * p.page_size + (w.pos % p.page_size)) * D;
    const bf16* krow = p.q + (size_t)tok * p.q_stride + (size_t)(p.nq + w.kvh) * D;
    const bf16* vrow = krow + (size_t)p.nkv * D;
    const bool mine = lane < D / 4;
    if (mine) reinterpret_cast<uint2*>(p.vpool + dst)[lane] = reinterpret_cast<const uint2*>(vrow)[lane];
    float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float ss = 0.0f;
    if (mine) {
        const uint2 raw = reinterpret_cast<const uint2*>(krow)[lane];
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
        ss += x[0] * x[0] + x[1] * x[1];
        ss += x[2] * x[2] + x[3] * x[3];
    }
    float inv = 1.0f;
    if (p.kw != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        inv = 1.0f / sqrtf(ss / (float)D + p.eps);
    }
    if (mine) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = p.kw != nullptr ? x[i] * inv * fd_weight(p.kw, p.w_f32, 4 * lane + i) : x[i];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int pr = 2 * lane + h;
            if (p.cos_t != nullptr && pr < p.rot_pairs) {
                const float c = p.cos_t[(size_t)tok * p.rot_pairs + pr], sn = p.sin_t[(size_t)tok * p.rot_pairs + pr];
                const float r0 = v[2 * h] * c - v[2 * h + 1] * sn;
                const float r1 = v[2 * h] * sn + v[2 * h + 1] * c;
                v[2 * h] = r0; v[2 * h + 1] = r1;
            }
        }
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a); raw.y = *reinterpret_cast<const unsigned*>(&b);
        reinterpret_cast<uint2*>(p.kpool + dst)[lane] = raw;
    }
}

// The pieces of a cut pair, added up in the order of their keys by the 128 softmax threads (thread = element of the
// head).  Piece i lies in the scratch of CTA cta_first + i: slot 1 there for the first one, slot 0 for the others.
// The loads of a chunk of pieces - maxima, sums and accumulators, for all heads of the group - are issued together
// (a chain of L2 latencies otherwise) and the chunks are folded into running sums that are rescaled when a later
// chunk brings a larger maximum: one pass over the scratch, the same arithmetic whatever the timing.
template <int D, int GP>
__device__ __forceinline__ void fd_merge(const FdParams& p, const FdItem& w, int tok, int tid, int G) {
    constexpr int PC = 32 / GP;          // pieces per chunk
    const int e = tid < D ? tid : 0;
    float mrun[GP], num[GP], den[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) { mrun[g] = -INFINITY; num[g] = 0.0f; den[g] = 0.0f; }
    for (int i0 = 0; i0 < w.pieces; i0 += PC) {
        float2 ml[PC][GP];
        float a[PC][GP];
#pragma unroll
        for (int i = 0; i < PC; ++i) {
            const size_t r = ((size_t)(w.cta_first + i0 + i) * 2 + (i0 + i == 0 ? 1 : 0)) * 16;
#pragma unroll
            for (int g = 0; g < GP; ++g) {
                const bool live = i0 + i < w.pieces && g < G;
                ml[i][g] = live ? __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (r + g) * 2)) : make_float2(-INFINITY, 0.0f);
                a[i][g] = live ? __ldcg(p.ws_acc + (r + g) * D + e) : 0.0f;
            }
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            float mnew = mrun[g];
#pragma unroll
            for (int i = 0; i < PC; ++i) mnew = fmaxf(mnew, ml[i][g].x);
            if (mnew == -INFINITY) continue;                       // nothing but masked keys so far
            const float keep = fa_ex2(mrun[g] - mnew);              // -inf gives 0
            num[g] *= keep;
            den[g] *= keep;
#pragma unroll
            for (int i = 0; i < PC; ++i) {
                const float f = fa_ex2(ml[i][g].x - mnew);
                num[g] += f * a[i][g];
                den[g] += f * ml[i][g].y;
            }
            mrun[g] = mnew;
        }
    }
    if (tid < D) {
#pragma unroll
        for (int g = 0; g < GP; ++g)
            if (g < G) {
                const size_t row = (size_t)tok * p.nq + (size_t)w.kvh * G + g;
                p.out[row * D + tid] = __float2bfloat16_rn(den[g] > 0.0f ? num[g] / den[g] : 0.0f);
            }
    }
}

// GP: the group's query heads rounded up to 4, 8 or 16
template <int D, int GP>
__global__ void __launch_bounds__(FD_THREADS, 1)
attn_decode_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const FdParams p) {
    constexpr int HALVES = D / 64;
    constexpr unsigned HALF_BYTES = 128 * 128;            // a 64-wide half of a key / value tile: 128 rows x 128 bytes
    constexpr unsigned TILE_BYTES = HALVES * HALF_BYTES;
    constexpr unsigned STAGE_BYTES = 2 * TILE_BYTES;      // keys, then values
    constexpr unsigned QHALF_BYTES = 16 * 128;            // 16 query rows x 128 bytes
    constexpr unsigned QBUF_BYTES = 2 * QHALF_BYTES;      // the queries of one item
    constexpr unsigned PHALF_BYTES = 16 * 128;            // 16 rows of probabilities x 64 keys
    constexpr unsigned TMEM_COLS = 64;                    // S^T twice (16 columns each), O^T (16 columns)
    constexpr unsigned O_COL = 32;
    constexpr int STAGES = FD_STAGES;
    constexpr int QCHUNKS = (GP * (D / 8) + 127) / 128;   // 16-byte pieces of the queries per softmax thread

    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* sKV = smem;                                        // [STAGES][K tile | V tile]
    unsigned char* sQ = sKV + STAGES * STAGE_BYTES;                   // [2 items][HALVES][16 rows][128 B]
    unsigned char* sP = sQ + 2 * QBUF_BYTES;                          // [2 halves of keys][16 rows][128 B]
    float* xmax = reinterpret_cast<float*>(sP + 2 * PHALF_BYTES);     // [2 parities][16 heads][4 warps]
    float* xsum = xmax + 2 * 16 * 4;                                  // [16 heads][4 warps]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(xsum + 16 * 4);
    unsigned long long* full = bars;                      // [STAGES] TMA -> MMA
    unsigned long long* empty = bars + STAGES;            // [STAGES] MMA -> TMA
    unsigned long long* s_full = bars + 2 * STAGES;       // [2] MMA -> softmax: scores of a tile
    unsigned long long* p_ready = s_full + 2;             // softmax (4 warps) -> MMA: P written, O rescaled, S read
    unsigned long long* pv_done = s_full + 3;             // MMA -> softmax: O updated, P free
    unsigned long long* q_ready = s_full + 4;             // [2] softmax (4 warps) -> MMA: an item's queries are in place
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(s_full + 6);
    volatile unsigned* failed = tmem_slot + 1;
    volatile int* merge_here = reinterpret_cast<volatile int*>(tmem_slot + 2);     // [2] softmax warps: this CTA adds the pieces of that pair up
    int* tokens_written = reinterpret_cast<int*>(tmem_slot + 4);                   // writer warp -> producer: pairs whose new token is in its page
    int* tile_pre = reinterpret_cast<int*>(tmem_slot + 6);                         // [FD_MAX_SEGS + 1] tiles, then [FD_MAX_SEGS + 1] segments

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.group;
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { fa_mbar_init(&full[i], 1); fa_mbar_init(&empty[i], 1); }
        fa_mbar_init(&s_full[0], 1); fa_mbar_init(&s_full[1], 1);
        fa_mbar_init(p_ready, 4); fa_mbar_init(pv_done, 1);
        fa_mbar_init(&q_ready[0], 4); fa_mbar_init(&q_ready[1], 4);
        *failed = 0;
        *tokens_written = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        // tiles per kv head, and single-token segments, before each segment: chunks of 32 segments, a warp scan in each.
        // The step's metadata was written before the kernels of this step began, so this does not wait for the previous one.
        int run = 0, run_d = 0;
        for (int s0 = 0; s0 < p.num_segments; s0 += 32) {
            const int sg = s0 + lane;
            const int n = sg < p.num_segments ? fd_seg_tiles(p, sg) : 0;
            const int dflag = n > 0 ? 1 : 0;
            int inc = n, inc_d = dflag;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, inc, o), up_d = __shfl_up_sync(0xffffffffu, inc_d, o);
                if (lane >= o) { inc += up; inc_d += up_d; }
            }
            if (sg < p.num_segments) { tile_pre[sg] = run + inc - n; tile_pre[FD_MAX_SEGS + 1 + sg] = run_d + inc_d - dflag; }
            run += __shfl_sync(0xffffffffu, inc, 31);
            run_d += __shfl_sync(0xffffffffu, inc_d, 31);
        }
        if (lane == 0) { tile_pre[p.num_segments] = run; tile_pre[FD_MAX_SEGS + 1 + p.num_segments] = run_d; }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_smem(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // ring, queries and probabilities start as zeros: rows that nothing fills (keys past the end of a pair's last tile,
    // query rows past the group) must not hold NaN bit patterns - a probability of exactly zero times a NaN is a NaN.
    // (Clearing only the value rows behind a pair's end, in the softmax threads, instead of the whole ring measured
    // the same step time.)
    for (unsigned i = threadIdx.x; i < (STAGES * STAGE_BYTES + 2 * QBUF_BYTES + 2 * PHALF_BYTES) / 16; i += FD_THREADS)
        reinterpret_cast<uint4*>(sKV)[i] = make_uint4(0, 0, 0, 0);
    pdl_wait();
    fa_fence_async_smem();
    fa_fence_before();
    __syncthreads();
    fa_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer: lane = page of the key tile; runs ahead across items ----------------
        const int ps = p.page_size, pages_per_tile = FA_BN / ps;
        const unsigned page_bytes = (unsigned)ps * 128u;
        int t = 0, newest_seen = 0;
        FdCursor cur;
        fd_begin(p, tile_pre, cur);
        FdItem w;
        bool ok = true;
        while (ok && !*failed && fd_next(p, tile_pre, cur, w)) {
            const int* table = p.block_table + (size_t)p.seg_slot[w.seg] * p.bt_stride;
            for (int j = 0; j < w.ntiles; ++j, ++t) {
                const int st = t % STAGES, use = t / STAGES;
                if (p.fuse && j == w.ntiles - 1 && w.newest) {
                    // the tile about to be requested holds the newest position: the writer warp must have put its key
                    // and value into the page (and made them visible to the TMA unit) first
                    ++newest_seen;
                    if (!fd_wait_count(tokens_written, newest_seen, (8u << 24) | t, failed)) { ok = false; break; }
                    __syncwarp();
                }
                const int key = w.kb + j * FA_BN + lane * ps;
                const int page = (lane < pages_per_tile && key < w.ke) ? table[key / ps] : -1;
                const unsigned mask = __ballot_sync(0xffffffffu, page >= 0);
                const unsigned bytes = (unsigned)__popc(mask) * page_bytes * HALVES * 2;
                const int row = (page * p.nkv + w.kvh) * ps;
                if (use > 0 && !fa_mbar_wait(&empty[st], (use - 1) & 1, (1u << 24) | t, failed)) { ok = false; break; }
                if (lane == 0) fa_mbar_expect_tx(&full[st], bytes);
                __syncwarp();
                if (page >= 0) {
                    unsigned char* dst = sKV + st * STAGE_BYTES + lane * page_bytes;
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        fa_tma_load(dst + h * HALF_BYTES, &map_k, h * 64, row, &full[st]);
                        fa_tma_load(dst + TILE_BYTES + h * HALF_BYTES, &map_v, h * 64, row, &full[st]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // S^T: M 128 keys x N 16 heads, both K-major.  O^T: M 128 (head dimension) x N 16, A (values) MN-major.
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            const unsigned idesc_pv = idesc_s | (1u << 15);
            int t = 0, ic = 0;
            FdCursor cur;
            fd_begin(p, tile_pre, cur);
            FdItem w;
            bool ok = true;
            auto issue_s = [&](int tt, int qbuf) -> bool {        // scores of tile tt into buffer tt & 1
                const int st = tt % STAGES;
                if (!fa_mbar_wait(&full[st], (tt / STAGES) & 1, (2u << 24) | tt, failed)) return false;
                fa_fence_after();
                const unsigned char* kt = sKV + st * STAGE_BYTES;
                const unsigned char* qt = sQ + qbuf * QBUF_BYTES;
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        fa_mma(tmem_base + (tt & 1) * 16, fa_desc_kmajor(fa_smem(kt + h * HALF_BYTES) + k * 32),
                               fa_desc_kmajor(fa_smem(qt + h * QHALF_BYTES) + k * 32), idesc_s, (h > 0 || k > 0) ? 1u : 0u);
                fa_commit(&s_full[tt & 1]);
                return true;
            };
            while (ok && !*failed && fd_next(p, tile_pre, cur, w)) {
                if (!fa_mbar_wait(&q_ready[ic & 1], (ic >> 1) & 1, (3u << 24) | ic, failed)) break;
                const int qbuf = ic & 1;
                ++ic;
                ok = issue_s(t, qbuf);
                for (int j = 0; j < w.ntiles && ok; ++j, ++t) {
                    if (j + 1 < w.ntiles) ok = issue_s(t + 1, qbuf);      // the next scores while this tile is in its softmax
                    if (!ok) break;
                    if (!fa_mbar_wait(p_ready, t & 1, (4u << 24) | t, failed)) { ok = false; break; }
                    fa_fence_after();
                    const int st = t % STAGES;
                    const unsigned char* vt = sKV + st * STAGE_BYTES + TILE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < FA_BN / 16; ++kk)
                        fa_mma(tmem_base + O_COL, fa_desc_mnmajor(fa_smem(vt) + kk * 16 * 128, HALVES == 2 ? HALF_BYTES : 0u),
                               fa_desc_kmajor(fa_smem(sP + (kk / 4) * PHALF_BYTES) + (kk % 4) * 32), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
                    fa_commit(pv_done);
                    fa_commit(&empty[st]);        // keys and values of this stage are no longer read
                }
            }
        }
    } else if (warp == 6) {
        // ---------------- writer of the new tokens (fused mode): ahead of the producer, pair by pair ----------------
        if (p.fuse) {
            FdCursor cur;
            fd_begin(p, tile_pre, cur);
            FdItem w;
            int done = 0;
            while (!*failed && fd_next(p, tile_pre, cur, w)) {
                if (!w.newest) continue;
                const int* table = p.block_table + (size_t)p.seg_slot[w.seg] * p.bt_stride;
                fd_write_new_token<D>(p, w, table, lane);
                // visible to the TMA unit (proxy fence by the writers), then the warp meets and says so
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __syncwarp();
                ++done;
                if (lane == 0) fd_set_count(tokens_written, done);
            }
        }
    } else {
        // ---------------- softmax and output: thread = key (scores) / = element of the head (output) ----------------
        const int quarter = warp & 3;
        const int tid = quarter * 32 + lane;               // TMEM lane of this thread
        const unsigned lane_base = (unsigned)(quarter * 32) << 16;
        int t = 0, ic = 0;
        bool alive = true;
        // the queries of an item: rows g < G of a [16, D] K-major tile; fetched into registers early, stored later
        uint4 qv[QCHUNKS];
        auto fetch_q = [&](const FdItem& w) {
            const int tok = p.seg_off[w.seg];
#pragma unroll
            for (int c = 0; c < QCHUNKS; ++c) {
                const int idx = tid + c * 128;
                qv[c] = make_uint4(0, 0, 0, 0);
                if (idx < G * (D / 8))
                    qv[c] = *reinterpret_cast<const uint4*>(p.q + (size_t)tok * p.q_stride + (size_t)(w.kvh * G + idx / (D / 8)) * D + (idx % (D / 8)) * 8);
            }
        };
        // fused mode: the raw queries become normalised, rotated ones.  A head's D elements sit in D / 8 neighbouring
        // threads (8 elements each); threads beyond the group's heads hold zeros and only take part in the shuffles.
        auto finish_q = [&](const FdItem& w) {
            if (!p.fuse) return;
            const int tok = p.seg_off[w.seg];
#pragma unroll
            for (int c = 0; c < QCHUNKS; ++c) {
                const int idx = tid + c * 128;
                const int ch = idx % (D / 8);
                float x[8];
                {
                    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&qv[c]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { x[2 * i] = __low2float(h2[i]); x[2 * i + 1] = __high2float(h2[i]); }
                }
                float inv = 1.0f;
                if (p.qw != nullptr) {
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
                    for (int o = D / 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    inv = 1.0f / sqrtf(ss / (float)D + p.eps);
                }
                if (idx < G * (D / 8)) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (p.qw != nullptr) x[i] = x[i] * inv * fd_weight(p.qw, p.w_f32, 8 * ch + i);
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const int pr = 4 * ch + h;
                        if (p.cos_t != nullptr && pr < p.rot_pairs) {
                            const float cs = p.cos_t[(size_t)tok * p.rot_pairs + pr], sn = p.sin_t[(size_t)tok * p.rot_pairs + pr];
                            const float r0 = x[2 * h] * cs - x[2 * h + 1] * sn;
                            const float r1 = x[2 * h] * sn + x[2 * h + 1] * cs;
                            x[2 * h] = r0; x[2 * h + 1] = r1;
                        }
                    }
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&qv[c]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
                }
            }
        };
        auto store_q = [&](int buf) {
#pragma unroll
            for (int c = 0; c < QCHUNKS; ++c) {
                const int idx = tid + c * 128;
                if (idx < G * (D / 8)) {
                    const int g = idx / (D / 8), ch = idx % (D / 8);
                    *reinterpret_cast<uint4*>(sQ + buf * QBUF_BYTES + (ch / 8) * QHALF_BYTES + g * 128 + (((ch % 8) ^ (g & 7)) << 4)) = qv[c];
                }
            }
            fa_fence_async_smem();
            __syncwarp();
            if (lane == 0) fa_mbar_arrive(&q_ready[buf]);
        };
        FdItem w, wn;
        FdItem cut[2];               // pieces of cut pairs that this CTA has left in the scratch
        int cut_tok[2], ncut = 0;
        FdCursor cur;
        fd_begin(p, tile_pre, cur);
        bool have = fd_next(p, tile_pre, cur, w);
        if (have) { fetch_q(w); finish_q(w); store_q(0); }
        while (have) {
            const bool have_next = fd_next(p, tile_pre, cur, wn);
            if (have_next) fetch_q(wn);                    // lands while this item's first tile is worked on
            const int tok = p.seg_off[w.seg];
            float m_run[GP], l_thr[GP];
#pragma unroll
            for (int g = 0; g < GP; ++g) { m_run[g] = -INFINITY; l_thr[g] = 0.0f; }
            for (int j = 0; j < w.ntiles; ++j, ++t) {
                alive = alive && fa_mbar_wait(&s_full[t & 1], (t >> 1) & 1, (5u << 24) | t, failed);
                fa_fence_after();
                float s[GP];
                fa_tmem_ld_cols<GP>(tmem_base + (t & 1) * 16 + lane_base, s);
                const int key = w.kb + j * FA_BN + tid;
                const bool vis = key <= w.pos && key >= w.lo && key < w.ke;
                float* xm = xmax + (t & 1) * 64;
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                    s[g] = vis ? s[g] * p.scale_log2 : -INFINITY;
                    const float wm = fa_warp_max(s[g]);
                    if (lane == 0) xm[g * 4 + quarter] = wm;
                }
                fd_softmax_sync();
                float alpha[GP];
                bool moved = false;
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                    const float4 q4 = *reinterpret_cast<const float4*>(xm + g * 4);
                    const float m_new = fmaxf(m_run[g], fmaxf(fmaxf(q4.x, q4.y), fmaxf(q4.z, q4.w)));
                    const float base = (m_new == -INFINITY) ? 0.0f : m_new;
                    alpha[g] = fa_ex2(m_run[g] - base);
                    moved = moved || (alpha[g] != 1.0f);
                    m_run[g] = m_new;
                    s[g] = fa_ex2(s[g] - base);                 // -inf gives 0
                    l_thr[g] = l_thr[g] * alpha[g] + s[g];
                }
                // the previous P V of this item must be complete before P is overwritten and O rescaled
                if (j > 0) alive = alive && fa_mbar_wait(pv_done, (t - 1) & 1, (6u << 24) | t, failed);
                fa_fence_after();
                {
                    unsigned char* pcol = sP + (tid >> 6) * PHALF_BYTES + ((tid & 7) << 1);
                    const int chunk = (tid & 63) >> 3;
#pragma unroll
                    for (int g = 0; g < GP; ++g)
                        if (g < G) *reinterpret_cast<bf16*>(pcol + g * 128 + ((chunk ^ (g & 7)) << 4)) = __float2bfloat16_rn(s[g]);
                }
                if (j > 0 && moved) {      // the same decision in every thread: the maxima are the same
                    float o[GP];
                    fa_tmem_ld_cols<GP>(tmem_base + O_COL + lane_base, o);
#pragma unroll
                    for (int g = 0; g < GP; ++g) o[g] *= alpha[g];
                    fa_tmem_st_cols<GP>(tmem_base + O_COL + lane_base, o);
                }
                fa_fence_before();
                fa_fence_async_smem();
                __syncwarp();
                if (lane == 0) fa_mbar_arrive(p_ready);
                if (j == 0 && have_next) { finish_q(wn); store_q((ic + 1) & 1); }     // the next item's queries, fetched above
            }
            // ---------------- the piece's result ----------------
            alive = alive && fa_mbar_wait(pv_done, (t - 1) & 1, (7u << 24) | t, failed);
            fa_fence_after();
            float o[GP];
            fa_tmem_ld_cols<GP>(tmem_base + O_COL + lane_base, o);
            fa_fence_before();
#pragma unroll
            for (int g = 0; g < GP; ++g) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) l_thr[g] += __shfl_xor_sync(0xffffffffu, l_thr[g], off);
                if (lane == 0) xsum[g * 4 + quarter] = l_thr[g];
            }
            fd_softmax_sync();
            if (alive) {
                const size_t ws_row = ((size_t)blockIdx.x * 2 + w.slot) * 16;
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                    if (g < G) {
                        const float4 q4 = *reinterpret_cast<const float4*>(xsum + g * 4);
                        const float l = (q4.x + q4.y) + (q4.z + q4.w);
                        if (w.whole) {
                            const size_t row = (size_t)tok * p.nq + (size_t)w.kvh * G + g;
                            if (tid < D) p.out[row * D + tid] = __float2bfloat16_rn(l > 0.0f ? o[g] / l : 0.0f);
                        } else {
                            if (tid < D) p.ws_acc[(ws_row + g) * D + tid] = o[g];
                            if (tid == 0) {
                                p.ws_ml[(ws_row + g) * 2] = m_run[g];
                                p.ws_ml[(ws_row + g) * 2 + 1] = l;
                            }
                        }
                    }
                }
            }
            if (!w.whole) {          // at most two per span: one that began before it, one that goes on behind it
                if (ncut == 0) { cut[0] = w; cut_tok[0] = tok; } else { cut[1] = w; cut_tok[1] = tok; }
                ++ncut;
            }
            fd_softmax_sync();            // xsum is read before the next piece overwrites it
            w = wn; have = have_next; ++ic;
        }
        // The span is done.  Its pieces of cut pairs are reported (writes, fence, then the count), and whoever reports
        // a pair's last piece adds them all up.  One thread takes the decisions for the four warps.
        if (ncut > 0) {
            __threadfence();
            fd_softmax_sync();
            if (tid == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (i >= ncut) break;
                    int last = 0;
                    if (alive) {
                        const unsigned before = atomicAdd(p.ws_count + cut[i].cta_first, 1u);
                        last = (before + 1u == (unsigned)cut[i].pieces) ? 1 : 0;
                        if (last) p.ws_count[cut[i].cta_first] = 0u;         // ready for the next launch
                    }
                    merge_here[i] = last;
                }
            }
            fd_softmax_sync();
#pragma unroll
            for (int i = 0; i < 2; ++i)
                if (i < ncut && merge_here[i]) {
                    __threadfence();
                    fd_merge<D, GP>(p, cut[i], cut_tok[i], tid, G);
                }
        }
    }
    // ---------------- common exit ----------------
    fa_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        fa_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

#ifdef FD_POISON_TEST
// Test builds only: every SM's shared memory is filled with NaN bit patterns, so that a kernel that reads shared
// memory it has not written shows it in its results.
__global__ void fd_poison_shared_kernel(unsigned bytes) {
    extern __shared__ unsigned char poison_smem[];
    for (unsigned i = threadIdx.x; i < bytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(poison_smem)[i] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
    __syncthreads();
    if (reinterpret_cast<volatile unsigned*>(poison_smem)[threadIdx.x] != 0xFFFFFFFFu) __nanosleep(1);      // keeps the stores
}
PI_EXPORT int pi_attention_tcgen05_test_poison_shared(cudaStream_t stream) {
    const unsigned bytes = 227 * 1024;
    cudaError_t err = cudaFuncSetAttribute(fd_poison_shared_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err != cudaSuccess) return (int)err;
    fd_poison_shared_kernel<<<4 * pi_sm_count(), 256, bytes, stream>>>(bytes);
    return pi_check_launch("pi_attention_tcgen05_test_poison_shared");
}
#endif

// ---- host side ---------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 fa_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

// the page pool as a [rows, D] bf16 matrix; boxes of page_size rows x 64 columns, 128-byte swizzle
static int fa_make_map(CUtensorMap* map, const void* base, long long rows, int page_size) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = fa_encode_fn();
    if (encode == nullptr) return pi_refuse("pi_attention_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)PI_HEAD_DIM, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)PI_HEAD_DIM * sizeof(bf16)};
    cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pi_refuse("pi_attention_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

PI_EXPORT int pi_attention_tcgen05_status(unsigned* status) {
    unsigned zero = 0;
    cudaError_t err = cudaMemcpyFromSymbol(status, g_fa_status, sizeof(unsigned));
    if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_fa_status, &zero, sizeof(unsigned));
    if (err != cudaSuccess) {
        snprintf(g_pi_error, sizeof(g_pi_error), "pi_attention_tcgen05_status: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return 0;
}

PI_EXPORT int pi_attention_tcgen05_supported(int page_size) {
    return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// Prompt portions only: segments of one token are skipped (run the decode kernel for those).
PI_EXPORT int pi_attention_tcgen05(const void* q, int q_stride, const void* kcache, const void* vcache, long long num_pages,
                                   const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                                   const int* seg_start, const int* seg_len, void* out, int num_segments, int max_seg_len,
                                   int nq, int nkv, int page_size, int window, float scale, int splits, float* part_acc,
                                   float* part_ml, const int* token_seg, int num_tokens, cudaStream_t stream) {
    if (num_segments <= 0 || max_seg_len <= 0) return 0;
    if (splits < 1 || splits > 64) return pi_refuse("pi_attention_tcgen05: splits=%d must be 1..64", splits);
    if (splits > 1 && (part_acc == nullptr || part_ml == nullptr || token_seg == nullptr || num_tokens <= 0))
        return pi_refuse("pi_attention_tcgen05: key splitting needs its scratch, the token-to-segment table and the token count");
    if (!(scale > 0.0f)) return pi_refuse("pi_attention_tcgen05: the score scale must be positive");
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) return pi_refuse("pi_attention_tcgen05: nq=%d must be a positive multiple of nkv=%d", nq, nkv);
    if (!pi_attention_tcgen05_supported(page_size)) return pi_refuse("pi_attention_tcgen05: page size %d is not one of 8, 16, 32, 64, 128", page_size);
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 127) || ((uintptr_t)vcache & 127))
        return pi_refuse("pi_attention_tcgen05: q must be 16-byte aligned with a stride that is a multiple of 8, pages 128-byte aligned");
    CUtensorMap mk, mv;
    const long long rows = num_pages * nkv * page_size;
    int rc = fa_make_map(&mk, kcache, rows, page_size);
    if (rc) return rc;
    rc = fa_make_map(&mv, vcache, rows, page_size);
    if (rc) return rc;
    FaParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.block_table = block_table; p.bt_stride = bt_stride;
    p.seg_off = seg_off; p.seg_slot = seg_slot; p.seg_start = seg_start; p.seg_len = seg_len;
    p.out = (bf16*)out; p.nq = nq; p.nkv = nkv; p.group = nq / nkv; p.page_size = page_size; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.tiles_per_seg = (int)(((long long)max_seg_len * p.group + FA_ROWS - 1) / FA_ROWS);
    p.num_segments = num_segments;
    p.splits = splits; p.part_acc = part_acc; p.part_ml = part_ml;
    const long long ctas = (long long)num_segments * p.tiles_per_seg * nkv;
    if (ctas > 2147483647LL) return pi_refuse("pi_attention_tcgen05: %lld tiles are beyond the grid limit", ctas);
    static bool configured = false;
    constexpr unsigned tile_bytes = (PI_HEAD_DIM / 64) * 128 * 128;
    const size_t smem = (size_t)(2 + FA_STAGES) * tile_bytes + (2 * FA_STAGES + 6) * 8 + 16 + 1024;
    auto kernel = attn_tcgen05_kernel<PI_HEAD_DIM>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "pi_attention_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    pi_launch(kernel, dim3((unsigned)ctas, (unsigned)splits), dim3(FA_THREADS), smem, stream, mk, mv, p);
    rc = pi_check_launch("pi_attention_tcgen05");
    if (rc || splits == 1) return rc;
    pi_launch(attn_prompt_merge_kernel<PI_HEAD_DIM>, dim3((unsigned)((long long)num_tokens * nq)), dim3(PI_HEAD_DIM), 0, stream,
              (const float*)part_acc, (const float*)part_ml, splits, (bf16*)out, token_seg, seg_len, nq);
    return pi_check_launch("pi_attention_tcgen05 merge");
}


PI_EXPORT int pi_attention_decode_tcgen05_supported(int page_size, int group) {
    return (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64) && group >= 1 && group <= 16;
}

// Segments of one token only (the others are skipped).  The workspace serves the pairs that are cut between CTAs:
// ws_acc [ws_ctas * 2 * 16 * D] and ws_ml [ws_ctas * 2 * 16 * 2] floats need no initial contents; ws_count [ws_ctas]
// must be zero before the first launch and is left zero by every launch that ends without a failed wait.  Launches
// that share a workspace must not overlap.  The kernel runs on min(SMs, ws_ctas) CTAs.
// what the fused form needs beside the arguments of pi_attention_decode_tcgen05
struct FdFusion {
    int fuse;
    const void* qw; const void* kw; int w_f32; float eps;
    const float* cos_t; const float* sin_t; int rot_pairs;
    int* error_count;
};

static int fd_launch(const void* q, int q_stride, const void* kcache, const void* vcache, long long num_pages,
                     const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                     const int* seg_start, const int* seg_len, void* out, float* ws_acc, float* ws_ml,
                     unsigned* ws_count, int ws_ctas, int span_min, int pair_cost, int num_segments, int nq, int nkv, int page_size,
                     int window, float scale, const FdFusion& fusion, cudaStream_t stream) {
    if (num_segments <= 0) return 0;
    if (!(scale > 0.0f)) return pi_refuse("pi_attention_decode_tcgen05: the score scale must be positive");
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0) return pi_refuse("pi_attention_decode_tcgen05: nq=%d must be a positive multiple of nkv=%d", nq, nkv);
    if (!pi_attention_decode_tcgen05_supported(page_size, nq / nkv))
        return pi_refuse("pi_attention_decode_tcgen05: page size %d must be 8, 16, 32 or 64 and the group (%d) at most 16", page_size, nq / nkv);
    if (num_segments > FD_MAX_SEGS) return pi_refuse("pi_attention_decode_tcgen05: %d segments; this kernel takes at most %d", num_segments, FD_MAX_SEGS);
    if (ws_ctas < 1 || ws_acc == nullptr || ws_ml == nullptr || ws_count == nullptr)
        return pi_refuse("pi_attention_decode_tcgen05: the workspace (for %d CTAs) is missing", ws_ctas);
    if (span_min < 1 || pair_cost < 0 || pair_cost > 64)
        return pi_refuse("pi_attention_decode_tcgen05: span_min=%d must be at least 1 and pair_cost=%d between 0 and 64", span_min, pair_cost);
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 127) || ((uintptr_t)vcache & 127))
        return pi_refuse("pi_attention_decode_tcgen05: q must be 16-byte aligned with a stride that is a multiple of 8, pages 128-byte aligned");
    CUtensorMap mk, mv;
    const long long rows = num_pages * nkv * page_size;
    int rc = fa_make_map(&mk, kcache, rows, page_size);
    if (rc) return rc;
    rc = fa_make_map(&mv, vcache, rows, page_size);
    if (rc) return rc;
    // the longest sequence of tiles the 32-bit cursors may meet: every segment at the last position a block table row holds
    const long long tiles_bound = (long long)num_segments * nkv * (((long long)bt_stride * page_size + FA_BN - 1) / FA_BN + 1 + pair_cost);
    if (tiles_bound > 2147483647LL / 2) return pi_refuse("pi_attention_decode_tcgen05: up to %lld key tiles are beyond the limit", tiles_bound);
    FdParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.block_table = block_table; p.bt_stride = bt_stride;
    p.seg_off = seg_off; p.seg_slot = seg_slot; p.seg_start = seg_start; p.seg_len = seg_len;
    p.out = (bf16*)out; p.ws_acc = ws_acc; p.ws_ml = ws_ml; p.ws_count = ws_count; p.span_min = span_min; p.pair_cost = pair_cost;
    p.nq = nq; p.nkv = nkv; p.group = nq / nkv; p.page_size = page_size; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.num_segments = num_segments;
    p.fuse = fusion.fuse; p.kpool = (bf16*)kcache; p.vpool = (bf16*)vcache;
    p.qw = fusion.qw; p.kw = fusion.kw; p.w_f32 = fusion.w_f32; p.eps = fusion.eps;
    p.cos_t = fusion.cos_t; p.sin_t = fusion.sin_t; p.rot_pairs = fusion.rot_pairs; p.error_count = fusion.error_count;
    static int sms = 0;
    static bool configured = false;
    constexpr unsigned tile_bytes = (PI_HEAD_DIM / 64) * 128 * 128;
    const size_t smem = (size_t)FD_STAGES * 2 * tile_bytes + 6 * 16 * 128 + (2 * 4 * 16 + 4 * 16) * 4 + (2 * FD_STAGES + 6) * 8 + 32 +
                        2 * (FD_MAX_SEGS + 1) * 4 + 1024;
    if (!configured) {
        int dev = 0;
        cudaError_t err = cudaGetDevice(&dev);
        if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "pi_attention_decode_tcgen05: cannot set up (%zu bytes of shared memory): %s", smem, cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    const unsigned ctas = (unsigned)(ws_ctas < sms ? ws_ctas : sms);
    if (p.group <= 4) pi_launch(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 4>, dim3(ctas), dim3(FD_THREADS), smem, stream, mk, mv, p);
    else if (p.group <= 8) pi_launch(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 8>, dim3(ctas), dim3(FD_THREADS), smem, stream, mk, mv, p);
    else pi_launch(attn_decode_tcgen05_kernel<PI_HEAD_DIM, 16>, dim3(ctas), dim3(FD_THREADS), smem, stream, mk, mv, p);
    return pi_check_launch("pi_attention_decode_tcgen05");
}

PI_EXPORT int pi_attention_decode_tcgen05(const void* q, int q_stride, const void* kcache, const void* vcache, long long num_pages,
                                          const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                                          const int* seg_start, const int* seg_len, void* out, float* ws_acc, float* ws_ml,
                                          unsigned* ws_count, int ws_ctas, int span_min, int pair_cost, int num_segments, int nq, int nkv,
                                          int page_size, int window, float scale, cudaStream_t stream) {
    const FdFusion none = {0, nullptr, nullptr, 0, 0.0f, nullptr, nullptr, 0, nullptr};
    return fd_launch(q, q_stride, kcache, vcache, num_pages, block_table, bt_stride, seg_off, seg_slot, seg_start, seg_len, out,
                     ws_acc, ws_ml, ws_count, ws_ctas, span_min, pair_cost, num_segments, nq, nkv, page_size, window, scale, none, stream);
}

// The same for a step of single tokens straight from the q/k/v product: `qkv` [T, q_stride] holds nq query heads,
// nkv key heads and nkv value heads per token, all raw.  Per-head RMSNorm of queries and keys (weights q_weight /
// k_weight [D] in bf16 or float32 (weight_dtype), eps; both null: no norm), rotation of adjacent pairs (2i, 2i + 1)
// by cos_t / sin_t [T, rot_pairs] (null: none) and the write of every token's key and value into its page happen
// inside the attention kernel; no other kernel has to touch qkv or the pages for these tokens.  A token whose page
// is missing is counted in *error_count and not written.  Every segment must be a single token.
PI_EXPORT int pi_attention_decode_tcgen05_fused(const void* qkv, int q_stride, void* kcache, void* vcache, long long num_pages,
                                                const int* block_table, int bt_stride, const int* seg_off, const int* seg_slot,
                                                const int* seg_start, const int* seg_len, void* out, float* ws_acc,
                                                float* ws_ml, unsigned* ws_count, int ws_ctas, int span_min, int pair_cost, int num_segments,
                                                int nq, int nkv, int page_size, int window, float scale, const void* q_weight,
                                                const void* k_weight, int weight_dtype, float eps, const float* cos_t,
                                                const float* sin_t, int rot_pairs, int* error_count, cudaStream_t stream) {
    if ((q_weight == nullptr) != (k_weight == nullptr)) return pi_refuse("pi_attention_decode_tcgen05_fused: give both norm weights or none");
    if (q_weight != nullptr && weight_dtype != PI_F32 && weight_dtype != PI_BF16)
        return pi_refuse("pi_attention_decode_tcgen05_fused: unknown dtype code %d of the norm weights", weight_dtype);
    if ((cos_t == nullptr) != (sin_t == nullptr) || rot_pairs < 0 || rot_pairs * 2 > PI_HEAD_DIM)
        return pi_refuse("pi_attention_decode_tcgen05_fused: rotation tables / rot_pairs=%d do not fit head size %d", rot_pairs, PI_HEAD_DIM);
    if (error_count == nullptr) return pi_refuse("pi_attention_decode_tcgen05_fused: error_count is needed");
    if (q_stride < (nq + 2 * nkv) * PI_HEAD_DIM) return pi_refuse("pi_attention_decode_tcgen05_fused: rows of %d elements cannot hold %d + 2 x %d heads", q_stride, nq, nkv);
    const FdFusion fusion = {1, q_weight, k_weight, weight_dtype == PI_F32 ? 1 : 0, eps, cos_t, sin_t, rot_pairs, error_count};
    return fd_launch(qkv, q_stride, kcache, vcache, num_pages, block_table, bt_stride, seg_off, seg_slot, seg_start, seg_len, out,
                     ws_acc, ws_ml, ws_count, ws_ctas, span_min, pair_cost, num_segments, nq, nkv, page_size, window, scale, fusion, stream);
}

#else   // head sizes this kernel does not take

PI_EXPORT int pi_attention_tcgen05_supported(int page_size) { (void)page_size; return 0; }
PI_EXPORT int pi_attention_decode_tcgen05_supported(int page_size, int group) { (void)page_size; (void)group; return 0; }

#endif

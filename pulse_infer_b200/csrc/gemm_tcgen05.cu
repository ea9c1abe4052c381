// Matrix product on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T, bfloat16 operands,
// 32-bit accumulation in tensor memory (TMEM), bfloat16 or float32 result, optionally with the gated
// activation of a SwiGLU feed-forward fused into the epilogue.
//
// Structure of a CTA (192 threads), persistent over output tiles of 128 x BN:
//   warp 0     one lane issues TMA loads (cp.async.bulk.tensor.2d) of a 128 x 64 tile of x and a BN x 64 tile
//              of W per pipeline stage into 128-byte-swizzled shared memory, signalled on an mbarrier
//   warp 1     allocates TMEM; one lane issues tcgen05.mma (M 128, N BN, K 16 per instruction, operands
//              described by shared-memory descriptors) and tcgen05.commit to free stages / publish the tile
//   warps 2-5  epilogue: tcgen05.ld of their 32-lane quarter of the accumulator, conversion, stores
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of a tile overlaps the
// main loop of the next one.
//
// Every wait on an mbarrier is bounded: after about a second of polling the kernel records where it gave up in
// a status word, stops waiting everywhere, frees its TMEM and returns; the host reads the status.
//
// Reference parity: the reference calls cublasGemmEx (CUDA_R_16BF, CUBLAS_COMPUTE_32F) for every product
// (src/ops/kernels/cuda/matmul_kernel.cu:132-154) with weights [out, in] used transposed
// (src/layer/linear.cpp:213), and runs SiLU and the product as separate kernels (src/model/qwen3/model.cpp:903-908).
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64            // 64 bf16 = 128 bytes = one swizzle row
#define TC_THREADS 192
#ifndef TC_SPIN_LIMIT
#define TC_SPIN_LIMIT (1u << 22)      // polls before a wait gives up (a test build sets a smaller number)
#endif

// ---- status word ---------------------------------------------------------------------------------------
// 0: fine.  Otherwise (code << 24) | detail of the first wait that ran out.
__device__ unsigned g_tc_status;

// ---- PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) if the barrier did not flip in time or another wait has
// already failed; callers then skip their work and fall through to the common exit.
__device__ __forceinline__ bool mbar_wait(void* bar, unsigned parity, unsigned code, volatile unsigned* failed) {
    for (unsigned spin = 0; spin < TC_SPIN_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023u) == 1023u && *failed) return false;
    }
    *failed = 1;
    atomicCAS(&g_tc_status, 0u, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, void* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tmem_alloc(void* dst_smem, unsigned cols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                          unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {   // arrives on `bar` when all MMAs issued so far have completed
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {   // 32 lanes x 32 columns: lane i gets its row
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

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64 bf16), 128-byte swizzle, 8-row
// groups 1024 bytes apart.  `addr` is the shared address of the (1024-byte aligned) tile plus the byte offset of
// the 16-element k step inside the swizzle row.
__device__ __forceinline__ unsigned long long umma_desc_sw128(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);          // start address, bits 0-13
    d |= (unsigned long long)1 << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= (unsigned long long)(1024 >> 4) << 32;                  // stride byte offset: 8 rows x 128 bytes
    d |= (unsigned long long)1 << 46;                            // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                            // 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n.
__device__ __forceinline__ unsigned umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
}

struct TcParams {
    void* out;
    int ldo;
    int M, N, K;
    int out_f32;     // 1: float32 output, 0: bfloat16
    int gated;       // 1: W rows come in blocks of 16, 8 gate features and their 8 up features; see the epilogue
    int tiles_m, tiles_n;
#ifdef TC_TEST_HOOKS
    int skip_load;   // test builds only: the pipeline iteration whose loads the producer leaves out (-1: none)
#endif
};

// One 32-column chunk of an accumulator row goes to memory: plain (bf16 or f32), or through the gated activation.
__device__ __forceinline__ void tc_store_chunk(const TcParams& p, int row, int col0, const float (&v)[32]) {
    if (p.gated) {
        // columns come in blocks of 16: 8 gate features followed by their 8 up features;
        // out[row, col0 / 2 + j] = silu(gate_j) * up_j  (out has N / 2 columns)
        const int col = col0 / 2;
        bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + col;
        alignas(16) bf16 packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g = v[(j >> 3) * 16 + (j & 7)], u = v[(j >> 3) * 16 + 8 + (j & 7)];
            packed[j] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
        }
        if (col + 16 <= p.N / 2 && (p.ldo & 7) == 0) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(packed);
            *reinterpret_cast<uint4*>(dst + 8) = *reinterpret_cast<const uint4*>(packed + 8);
        } else {
            for (int j = 0; j < 16 && col + j < p.N / 2; ++j) dst[j] = packed[j];
        }
    } else if (p.out_f32) {
        float* dst = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldo + col0;
        if (col0 + 32 <= p.N && (p.ldo & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = v[j];
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + col0;
        alignas(16) bf16 packed[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) packed[j] = __float2bfloat16_rn(v[j]);
        if (col0 + 32 <= p.N && (p.ldo & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(packed + j);
        } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = packed[j];
        }
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const TcParams p) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr unsigned TMEM_COLS = 2 * BN;                       // two accumulators
    static_assert(BN == 128 || BN == 256, "tile widths 128 and 256");
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;                                    // [STAGES][128 x 64 bf16]
    unsigned char* sB = smem + STAGES * A_BYTES;                 // [STAGES][BN x 64 bf16]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sB + STAGES * B_BYTES);
    unsigned long long* full = bars;                             // [STAGES] TMA -> MMA
    unsigned long long* empty = bars + STAGES;                   // [STAGES] MMA -> TMA
    unsigned long long* acc_full = bars + 2 * STAGES;            // [2] MMA -> epilogue
    unsigned long long* acc_empty = bars + 2 * STAGES + 2;       // [2] epilogue -> MMA
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * STAGES + 4);
    volatile unsigned* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;
    pdl_wait();     // x is produced by the previous kernel

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int k_tiles = (p.K + TC_BK - 1) / TC_BK;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            unsigned it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * TC_BM, n0 = (tile / p.tiles_m) * BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const unsigned s = it % STAGES, round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, (1u << 24) | it, failed)) break;
#ifdef TC_TEST_HOOKS
                    if ((int)it == p.skip_load) continue;      // nothing will ever complete this stage: the consumer's wait runs out
#endif
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    tma_load_2d(sA + s * A_BYTES, &map_x, kt * TC_BK, m0, &full[s]);
                    tma_load_2d(sB + s * B_BYTES, &map_w, kt * TC_BK, n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const unsigned idesc = umma_idesc(BN);
            unsigned it = 0, local = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x, ++local) {
                const unsigned a = local & 1, use = local >> 1;        // accumulator buffer and how often it was used
                if (use > 0 && !mbar_wait(&acc_empty[a], (use - 1) & 1, (2u << 24) | local, failed)) break;
                tc_fence_after();
                const unsigned tmem_d = tmem_base + a * BN;
                bool ok = true;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const unsigned s = it % STAGES, round = it / STAGES;
                    if (!mbar_wait(&full[s], round & 1, (3u << 24) | it, failed)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(sA + s * A_BYTES), b_addr = smem_u32(sB + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16(tmem_d, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                                  (kt > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);                            // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[a]);                             // the tile is complete once all MMAs have finished
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31 ----------------
        const int quarter = warp & 3;
        unsigned local = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x, ++local) {
            const unsigned a = local & 1, use = local >> 1;
            if (!mbar_wait(&acc_full[a], use & 1, (4u << 24) | local, failed)) break;
            tc_fence_after();
            const int m0 = (tile % p.tiles_m) * TC_BM, n0 = (tile / p.tiles_m) * BN;
            const int row = m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + a * BN + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                tmem_ld32(taddr + c, v);
                if (row < p.M) tc_store_chunk(p, row, n0 + c, v);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[a]);                 // 4 arrivals (one per epilogue warp) free the buffer
        }
    }
    // ---------------- common exit ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------
// The same product on CTA pairs (cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile.  Each CTA
// loads its own 128 rows of x and its own half (128 rows) of the W tile; one thread of the pair's first CTA
// issues tcgen05.mma.cta_group::2 (M 256), which reads both CTAs' shared memory and writes rows 0-127 of the
// tile into its own TMEM and rows 128-255 into the peer's.  Per CTA that is 32 KB of operands per 64-wide k
// step instead of 48 KB for the same tensor-core work.  No multicast loads are used: readiness of the peer's
// stage reaches the first CTA by a forwarding thread (wait on the own barrier, remote arrive on the leader's).
// tcgen05.commit multicasts "stage free" and "tile complete" to both CTAs.
// Threads: warp 0 TMA, warp 1 MMA (leader only) + TMEM, warps 2-5 epilogue, warp 6 forwarder (peer only).
// ---------------------------------------------------------------------------------------------------
#define TC2_THREADS 192

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(void* bar, unsigned cta) {   // arrive on the same barrier of CTA `cta`
    unsigned raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(bar)), "r"(cta));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(raddr) : "memory");
}
__device__ __forceinline__ unsigned mapa_u32(void* ptr, unsigned cta) {
    unsigned raddr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(raddr) : "r"(smem_u32(ptr)), "r"(cta));
    return raddr;
}
// TMA load into this CTA's shared memory whose completion bytes are reported to a barrier of the CTA pair
// (given as a shared::cluster address, here the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, unsigned bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(void* dst_smem, unsigned cols) {    // one warp in each CTA of the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma2_bf16(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                           unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_commit_both(void* bar) {   // arrives on `bar` in both CTAs of the pair
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(TC2_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const TcParams p) {
    constexpr int BN = 256, HALF = 128;
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = HALF * TC_BK * 2;
    constexpr unsigned TMEM_COLS = 2 * BN;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* sA = smem;                                    // [STAGES][128 x 64 bf16] this CTA's rows of x
    unsigned char* sB = smem + STAGES * A_BYTES;                 // [STAGES][128 x 64 bf16] this CTA's half of the W tile
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sB + STAGES * B_BYTES);
    unsigned long long* full = bars;                             // [STAGES] leader only: both CTAs' loads of the stage landed
    unsigned long long* peer_full = bars + STAGES;               // [STAGES] unused (kept so that both kernels share a layout)
    unsigned long long* empty = bars + 2 * STAGES;               // [STAGES] MMA (multicast) -> both producers
    unsigned long long* acc_full = bars + 3 * STAGES;            // [2] MMA (multicast) -> both epilogues
    unsigned long long* acc_empty = bars + 3 * STAGES + 2;       // [2] leader only: 8 epilogue warps of the pair
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 3 * STAGES + 4);
    volatile unsigned* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();                        // 0: leader (issues the MMAs), 1: peer
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&peer_full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc2(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                          // both CTAs' barriers exist before anyone signals them
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    const int pairs = gridDim.x / 2, pair = blockIdx.x / 2;
    const int num_tiles = p.tiles_m * p.tiles_n;                 // tiles of 256 x 256
    const int k_tiles = (p.K + TC_BK - 1) / TC_BK;

    if (warp == 0) {
        if (lane == 0) {
            unsigned it = 0;
            for (int tile = pair; tile < num_tiles && !*failed; tile += pairs) {
                const int m0 = (tile % p.tiles_m) * 256 + (int)rank * TC_BM, n0 = (tile / p.tiles_m) * BN + (int)rank * HALF;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const unsigned s = it % STAGES, round = it / STAGES;
                    if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1, (1u << 24) | it, failed)) break;
                    if (rank == 0) {
                        mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));      // this CTA's bytes and the peer's
                        tma_load_2d(sA + s * A_BYTES, &map_x, kt * TC_BK, m0, &full[s]);
                        tma_load_2d(sB + s * B_BYTES, &map_w, kt * TC_BK, n0, &full[s]);
                    } else {
                        const unsigned leader_full = mapa_u32(&full[s], 0);
                        tma_load_2d_pair(sA + s * A_BYTES, &map_x, kt * TC_BK, m0, leader_full);
                        tma_load_2d_pair(sB + s * B_BYTES, &map_w, kt * TC_BK, n0, leader_full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
            unsigned it = 0, local = 0;
            for (int tile = pair; tile < num_tiles && !*failed; tile += pairs, ++local) {
                const unsigned a = local & 1, use = local >> 1;
                if (use > 0 && !mbar_wait(&acc_empty[a], (use - 1) & 1, (2u << 24) | local, failed)) break;
                tc_fence_after();
                const unsigned tmem_d = tmem_base + a * BN;
                bool ok = true;
                for (int kt = 0; kt < k_tiles; ++kt, ++it) {
                    const unsigned s = it % STAGES, round = it / STAGES;
                    if (!mbar_wait(&full[s], round & 1, (3u << 24) | it, failed)) { ok = false; break; }
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(sA + s * A_BYTES), b_addr = smem_u32(sB + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma2_bf16(tmem_d, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                                   (kt > 0 || k > 0) ? 1u : 0u);
                    umma2_commit_both(&empty[s]);
                }
                if (!ok) break;
                umma2_commit_both(&acc_full[a]);
            }
        }
    } else {
        const int quarter = warp & 3;
        unsigned local = 0;
        for (int tile = pair; tile < num_tiles && !*failed; tile += pairs, ++local) {
            const unsigned a = local & 1, use = local >> 1;
            if (!mbar_wait(&acc_full[a], use & 1, (4u << 24) | local, failed)) break;
            tc_fence_after();
            const int m0 = (tile % p.tiles_m) * 256 + (int)rank * TC_BM, n0 = (tile / p.tiles_m) * BN;
            const int row = m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + a * BN + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                tmem_ld32(taddr + c, v);
                if (row < p.M) tc_store_chunk(p, row, n0 + c, v);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&acc_empty[a]);
                else mbar_arrive_remote(&acc_empty[a], 0);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();          // nobody frees TMEM or leaves while the pair may still touch its memory or barriers
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc2(tmem_base, TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 tc_encode_fn() {
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

// rows x K bf16 matrix with row stride ld (elements); boxes of box_rows x 64 elements, 128-byte swizzle
static int tc_make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = tc_encode_fn();
    if (encode == nullptr) return pi_refuse("pi_gemm_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return pi_refuse("pi_gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int BN, int STAGES>
static int tc_launch(const CUtensorMap& mx, const CUtensorMap& mw, const TcParams& p, int ctas, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + (2 * STAGES + 4) * 8 + 16 + 1024;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "pi_gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    pi_launch(kernel, dim3(ctas), dim3(TC_THREADS), smem, stream, mx, mw, p);
    return pi_check_launch("pi_gemm_tcgen05");
}

template <int STAGES>
static int tc_launch_2cta(const CUtensorMap& mx, const CUtensorMap& mw, const TcParams& p, int pairs, cudaStream_t stream) {
    static bool configured = false;
    const size_t smem = (size_t)STAGES * (TC_BM + 128) * TC_BK * 2 + (3 * STAGES + 4) * 8 + 16 + 1024;
    auto kernel = gemm_tcgen05_2cta_kernel<STAGES>;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) {
            snprintf(g_pi_error, sizeof(g_pi_error), "pi_gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
            return (int)err;
        }
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC2_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, mx, mw, p);
    return pi_check_launch("pi_gemm_tcgen05 (CTA pairs)");
}

// Reads and clears the status word of the last launches (synchronises the device).  0 means every wait was met.
PI_EXPORT int pi_gemm_tcgen05_status(unsigned* status) {
    unsigned zero = 0;
    cudaError_t err = cudaMemcpyFromSymbol(status, g_tc_status, sizeof(unsigned));
    if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(unsigned));
    if (err != cudaSuccess) {
        snprintf(g_pi_error, sizeof(g_pi_error), "pi_gemm_tcgen05_status: %s", cudaGetErrorString(err));
        return (int)err;
    }
    return 0;
}

#ifdef TC_TEST_HOOKS
// Test builds only (-DTC_TEST_HOOKS, never the library the engine loads): the next single-CTA launch leaves out
// the loads of pipeline iteration `it`, so that the wait for that stage runs out and the give-up path executes.
static int g_test_skip_load = -1;
PI_EXPORT void pi_gemm_tcgen05_test_skip_load(int it) { g_test_skip_load = it; }
PI_EXPORT unsigned pi_gemm_tcgen05_spin_limit() { return TC_SPIN_LIMIT; }
#endif

// gated = 1: W holds gate and up rows interleaved in blocks of 8 (rows 16b .. 16b+7 gate features 8b .. 8b+7,
// rows 16b+8 .. 16b+15 the matching up features); out is [M, N / 2] bf16 = silu(gate) * up.
// mode 0: CTA pairs when M > 128, single CTAs otherwise; 1: single CTAs; 2: CTA pairs
PI_EXPORT int pi_gemm_tcgen05(const void* x, int ldx, const void* W, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, int gated, int max_ctas, int mode, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
        return pi_refuse("pi_gemm_tcgen05: K=%d and the leading dimensions (%d, %d) must be positive multiples of 8", K, ldx, ldw);
    if (((uintptr_t)x | (uintptr_t)W) & 15) return pi_refuse("pi_gemm_tcgen05: operands must be 16-byte aligned");
    if (out_dtype != PI_F32 && out_dtype != PI_BF16) return pi_refuse("pi_gemm_tcgen05: unknown output dtype code %d", out_dtype);
    if (gated && (out_dtype != PI_BF16 || N % 16 != 0)) return pi_refuse("pi_gemm_tcgen05: the gated epilogue needs bf16 output and N %% 16 == 0 (N=%d)", N);
    const int BN = 256;
    const bool pairs_mode = mode == 2 || (mode == 0 && M > TC_BM);
    CUtensorMap mx, mw;
    int rc = tc_make_map(&mx, x, M, K, ldx, TC_BM);
    if (rc) return rc;
    rc = tc_make_map(&mw, W, N, K, ldw, pairs_mode ? 128 : BN);
    if (rc) return rc;
    TcParams p;
    p.out = out; p.ldo = ldo; p.M = M; p.N = N; p.K = K; p.out_f32 = out_dtype == PI_F32; p.gated = gated;
#ifdef TC_TEST_HOOKS
    p.skip_load = pairs_mode ? -1 : g_test_skip_load;
    g_test_skip_load = -1;
#endif
    if (pairs_mode) {
        p.tiles_m = (M + 255) / 256;
        p.tiles_n = (N + BN - 1) / BN;
        int pairs = p.tiles_m * p.tiles_n;
        const int limit = (max_ctas > 0 ? max_ctas : pi_sm_count()) / 2;
        if (pairs > limit) pairs = limit > 0 ? limit : 1;
        return tc_launch_2cta<6>(mx, mw, p, pairs, stream);
    }
    p.tiles_m = (M + TC_BM - 1) / TC_BM;
    p.tiles_n = (N + BN - 1) / BN;
    int ctas = p.tiles_m * p.tiles_n;
    const int limit = max_ctas > 0 ? max_ctas : pi_sm_count();
    if (ctas > limit) ctas = limit;
    return tc_launch<256, 4>(mx, mw, p, ctas, stream);
}

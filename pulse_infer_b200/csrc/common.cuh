// Shared helpers of the sm_100a kernels: exported-symbol macro, error reporting, dtype codes,
// conversions and warp/block reductions.  Every library built from these sources exports plain C
// functions that take raw device pointers and a stream; nothing here allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#define PI_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum { PI_F32 = 0, PI_BF16 = 1 };

typedef __nv_bfloat16 bf16;

// ---- error reporting -------------------------------------------------------------------------------
// Launchers return 0 on success, a positive cudaError_t, or -1 when they refuse their arguments; the
// text of the last refusal (or CUDA error) of this library is read with pi_last_error().
static char g_pi_error[512] = "";

static int pi_refuse(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
#include <stdarg.h>
static int pi_refuse(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_pi_error, sizeof(g_pi_error), fmt, ap);
    va_end(ap);
    return -1;
}

static int pi_check_launch(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        snprintf(g_pi_error, sizeof(g_pi_error), "%s: %s", what, cudaGetErrorString(err));
        return (int)err;
    }
    return 0;
}

PI_EXPORT const char* pi_last_error() { return g_pi_error; }

// ---- launching -------------------------------------------------------------------------------------
// Kernels are launched with "programmatic stream serialization": a kernel may be scheduled while the tail of
// the kernel before it (in the same stream) is still running, and waits at pdl_wait() until that kernel has
// completed and its writes are visible.  Everything a kernel does before pdl_wait() must therefore touch only
// memory that no earlier kernel of the step writes (weights); every kernel calls pdl_wait() before its first
// read of an activation and before its first write.  pdl_trigger() tells the runtime that the next kernel may
// be scheduled as soon as all CTAs of this one have started.  After a copy or a library kernel the attribute
// has no effect, and without it both calls do nothing.  PULSE_PDL=0 in the environment turns it off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Which kernels let their successor be scheduled early (bit mask): 1 small kernels, 2 products, 4 attention.
#ifndef PI_PDL_EARLY
#define PI_PDL_EARLY 3
#endif
#define PDL_SMALL 1
#define PDL_PRODUCT 2
#define PDL_ATTENTION 4
__device__ __forceinline__ void pdl_trigger(int kind = PDL_SMALL) {
    if (PI_PDL_EARLY & kind) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#include <stdlib.h>
static int pi_pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* env = getenv("PULSE_PDL");
        enabled = (env != nullptr && env[0] == '0') ? 0 : 1;
    }
    return enabled;
}

// Streaming multiprocessors of the current device (asked once); launch shapes are sized from it.
static int pi_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0, n = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
            return 1;
        sms = n;
    }
    return sms;
}

template <typename... Params, typename... Args>
static void pi_launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pi_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);   // an error is picked up by pi_check_launch
}

// ---- L2 prefetch of upcoming weights ------------------------------------------------------------------
// The small kernels between two weight-streaming products (norms, rotation, SiLU, attention merge) leave the
// memory system idle.  They can be launched with a few extra CTAs whose only job is to ask for the next
// product's weights to be brought into L2 (prefetch.global.L2, fire and forget), so that product starts on
// L2 hits instead of a cold pipe.  The extra CTAs sit after the kernel's own CTAs in blockIdx.x.
#define PI_PREFETCH_CTAS 96
#define PI_PREFETCH_MAX_BYTES (64ull << 20)
struct Prefetch {
    const char* ptr;
    unsigned long long bytes;   // 0: no prefetch CTAs were added
    int first_cta;              // blockIdx.x of the first prefetch CTA
};

static Prefetch pi_make_prefetch(const void* ptr, unsigned long long bytes, int own_ctas) {
    Prefetch pf;
    pf.ptr = (const char*)ptr;
    pf.bytes = ptr ? (bytes < PI_PREFETCH_MAX_BYTES ? bytes : PI_PREFETCH_MAX_BYTES) : 0;
    pf.first_cta = own_ctas;
    return pf;
}
static inline int pi_prefetch_ctas(const Prefetch& pf) { return pf.bytes ? PI_PREFETCH_CTAS : 0; }

// true: this CTA was a prefetch CTA (the caller returns)
__device__ __forceinline__ bool pi_prefetch_role(const Prefetch& pf) {
    if (pf.bytes == 0 || (int)blockIdx.x < pf.first_cta) return false;
    const unsigned long long lines = pf.bytes >> 7;   // 128-byte lines
    const unsigned long long stride = (unsigned long long)(gridDim.x - pf.first_cta) * blockDim.x;
    for (unsigned long long i = (unsigned long long)(blockIdx.x - pf.first_cta) * blockDim.x + threadIdx.x; i < lines; i += stride)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pf.ptr + (i << 7)));
    return true;
}

// ---- conversions -----------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions ------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the additions
// depends only on the block size, so a row's result does not depend on what else is in the launch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats of shared memory */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    float total = scratch[32];
    __syncthreads();
    return total;
}

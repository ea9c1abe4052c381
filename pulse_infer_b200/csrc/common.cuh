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

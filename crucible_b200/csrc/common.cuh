// Shared helpers for the kernels of this package: element conversion between
// float and bfloat16, reductions, and the launch-status convention.  Every
// exported launcher returns a cudaError_t as int (0 = success) and never
// synchronises; the caller passes the stream to launch on.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python wrappers
#define CB_F32 0
#define CB_BF16 1

// launcher-level refusals (not CUDA errors); Python turns them into messages
#define CB_ERR_UNSUPPORTED 100001

__device__ __forceinline__ float cb_to_float(float v) { return v; }
__device__ __forceinline__ float cb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T cb_from_float(float v);
template <> __device__ __forceinline__ float cb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float cb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float cb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  The
// order of the additions is fixed by the block size alone.
__device__ __forceinline__ float cb_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = cb_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

static inline int cb_last_error() { return (int)cudaGetLastError(); }

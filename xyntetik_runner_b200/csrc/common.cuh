// Shared helpers of the sm_100a kernels: dtype codes, conversions, reductions.
//
// Every launcher is `extern "C"`, takes raw device pointers, explicit extents
// and a stream, and returns 0 or a negative error code (see XR_ERR_*); the
// Python side turns a non-zero code into an exception.  No launcher
// allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define XR_F32 0
#define XR_BF16 1

#define XR_OK 0
#define XR_ERR_ARG (-1)        // a size or dtype the kernel refuses
#define XR_ERR_LAUNCH (-2)     // the runtime refused the launch (cudaGetLastError)

#define XR_EXPORT extern "C" __attribute__((visibility("default")))

static inline int xr_launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? XR_OK : XR_ERR_LAUNCH;
}

template <typename T> __device__ __forceinline__ float xr_to_f32(T v);
template <> __device__ __forceinline__ float xr_to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float xr_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T xr_from_f32(float v);
template <> __device__ __forceinline__ float xr_from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 xr_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float xr_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float xr_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on the block size, never on the data.
__device__ __forceinline__ float xr_block_sum(float v, float* scratch /* >= 33 floats */) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = xr_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? scratch[lane] : 0.f;
        t = xr_warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

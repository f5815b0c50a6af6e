// Shared device helpers of the sm_100a kernels: element types, warp and block
// reductions, launch error reporting.  Every kernel keeps its arithmetic in
// 32-bit floats; bfloat16 is a storage format only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Element type codes of the C interface.
#define ODIN_F32 0
#define ODIN_BF16 1

// Error codes of the C interface (0 = success, >0 = cudaError_t).
#define ODIN_ERR_UNSUPPORTED (-1)
#define ODIN_ERR_BAD_ARG (-2)
#define ODIN_ERR_TIMEOUT (-3)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// A weight vector that may be stored in either type (a tensor stored in
// 32-bit stays so, also beside bfloat16 activations).
struct VecRef {
    const void* p;
    int is_bf16;
    __device__ __forceinline__ float at(int i) const {
        return is_bf16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
    }
};

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

// Sum over a block of up to 1024 threads; `red` is 32 floats of shared memory.
// Every thread gets the result.  The order of the additions is fixed by the
// block size, so equal inputs give equal sums whatever else the grid holds.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

#define ODIN_LAUNCH_CHECK()                          \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

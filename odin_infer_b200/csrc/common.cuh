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

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through odin_launch may start
// while the kernel before it on the stream is still running; pdl_wait() blocks until
// that kernel has completed and its memory is visible.  Rules every kernel here keeps:
//   * pdl_trigger() first, so the next kernel's CTAs can take their places early;
//   * pdl_wait() before the first read of anything an earlier kernel wrote and before
//     the first global write (a buffer may be reused memory that an earlier kernel
//     still reads); before it a kernel may touch only what no kernel of the step writes:
//     weights and constant tables, the step's integer tables (the host copies them to the
//     device before the step's first kernel), and the cache as earlier steps left it;
//   * every kernel launched this way calls pdl_wait(), so completion stays in stream
//     order.  Set ODIN_PDL=0 in the environment to launch in plain stream order.
// ---------------------------------------------------------------------------
#ifdef ODIN_TRACE
// Kernel timeline for tuning (libraries built with ODIN_KERNEL_TRACE=1 only): thread 0 of every
// CTA records the time at which it starts and at which its wait for the previous kernel ends,
// as [time in ns, point << 56 | block size << 44 | grid size << 22 | block number] after a counter in word 0.
static __device__ unsigned long long* odin_trace_buf = nullptr;
static __device__ unsigned int odin_trace_cap = 0;
__device__ __forceinline__ void odin_trace_emit(unsigned long long point, unsigned long long t) {
    if (odin_trace_buf == nullptr) return;
    const unsigned long long idx = atomicAdd(odin_trace_buf, 1ULL);
    if (idx >= odin_trace_cap) return;
    const unsigned long long grid = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    const unsigned long long block = ((unsigned long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    odin_trace_buf[1 + 2 * idx] = t;
    odin_trace_buf[2 + 2 * idx] = (point << 56) | ((unsigned long long)blockDim.x << 44) | ((grid & 0x3fffff) << 22) | (block & 0x3fffff);
}
__device__ __forceinline__ unsigned long long odin_trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void odin_trace_mark(unsigned long long point, bool any_thread = false) {
    if ((!any_thread && (threadIdx.x | threadIdx.y | threadIdx.z) != 0) || odin_trace_buf == nullptr) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned long long idx = atomicAdd(odin_trace_buf, 1ULL);
    if (idx >= odin_trace_cap) return;
    const unsigned long long grid = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    const unsigned long long block = ((unsigned long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    odin_trace_buf[1 + 2 * idx] = t;
    odin_trace_buf[2 + 2 * idx] = (point << 56) | ((unsigned long long)blockDim.x << 44) | ((grid & 0x3fffff) << 22) | (block & 0x3fffff);
}
extern "C" __attribute__((weak)) int odin_trace_attach(void* buf, unsigned int cap) {
    if (cudaMemcpyToSymbol(odin_trace_buf, &buf, sizeof(buf)) != cudaSuccess) return 1;
    return cudaMemcpyToSymbol(odin_trace_cap, &cap, sizeof(cap)) != cudaSuccess;
}
#else
__device__ __forceinline__ void odin_trace_mark(unsigned long long, bool = false) {}
#endif

__device__ __forceinline__ void pdl_trigger() {
    odin_trace_mark(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    odin_trace_mark(1);
}

#include <cstdlib>
#include <cstring>

static inline bool odin_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("ODIN_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <typename... KArgs, typename... Args>
static inline void odin_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args&&... args) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = odin_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define ODIN_LAUNCH_CHECK()                          \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) return (int)e__;     \
    } while (0)

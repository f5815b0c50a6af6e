// Row-wise kernels: embedding gather, residual add fused with RMSNorm,
// SwiGLU, element type conversion.
//
// RMSNorm follows the reference's order of operations (infer/ops.odin:7-19):
//   ss = sum x^2; ss /= n; ss += eps; r = 1/sqrt(ss); o = w * (r * x)
// all in 32-bit.  The residual stream x is 32-bit in both precisions.
#include <type_traits>

#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int d, int V) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = (id >= 0 && id < V);
    const TW* row = table + (size_t)(ok ? id : 0) * d;
    float* o = out + (size_t)t * d;
    for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = ok ? to_f32(row[j]) : 0.f;
}

extern "C" int odin_embed(const void* table, int table_dtype, const int* ids, float* out,
                          int T, int d, int V, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == ODIN_BF16)
        odin_launch(embed_kernel<bf16>, dim3(T), dim3(threads), 0, s, (const bf16*)table, ids, out, d, V);
    else if (table_dtype == ODIN_F32)
        odin_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)table, ids, out, d, V);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------- residual add + RMSNorm
// One block per output row.  x_new = x + sum_s delta[s] (32-bit), written
// back to x when there is no row gather; out = w * (r * x_new).
// The sum of squares goes over the columns in an order fixed by the block
// size alone, so a row's result does not depend on the other rows.
template <typename TD>
__device__ __forceinline__ float4 load4(const TD* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 load4<bf16>(const bf16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

// Four consecutive weights (the index a multiple of 4, the vector 16-byte aligned).
__device__ __forceinline__ float4 load4w(const VecRef& w, int j) {
    return w.is_bf16 ? load4<bf16>((const bf16*)w.p + j) : load4<float>((const float*)w.p + j);
}

// VEC: the row length is a multiple of 4 and every pointer is 16-byte aligned, so the
// row moves in groups of four; the order of the additions per element (x, then the
// parts in order) and of the sum of squares per thread is the same in both variants.
// The loads of a group are issued together (eight parts at a time), so that a row costs
// one trip to memory and not one per part; the weights of the first group and the row
// number, which no earlier kernel writes, are fetched before the wait for that kernel.
template <typename TD, typename TO, bool VEC, int MAX_THREADS>
__device__ __forceinline__ void add_rmsnorm_body(float* __restrict__ x, const TD* __restrict__ delta, int n_split,
                                                 size_t split_stride, VecRef w, float eps, TO* __restrict__ out,
                                                 const int* __restrict__ rows, int d, float* red, float* rowbuf) {
    pdl_trigger();
    const int r = blockIdx.x;
    int src = r;
    if (rows != nullptr) src = rows[r];
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC && (int)threadIdx.x * 4 < d) w0 = load4w(w, threadIdx.x * 4);
    pdl_wait();
    TO* o = out + (size_t)r * d;
    if (src < 0) {
        for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_f32<TO>(0.f);
        return;
    }
    float* xr = x + (size_t)src * d;
    float ss = 0.f;
    if (VEC) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
            float4 v = load4<float>(xr + j);
            if (delta != nullptr) {
                const TD* dp = delta + (size_t)src * d + j;
                constexpr int BATCH = 2;  // loads in flight per thread (registers)
                for (int s0 = 0; s0 < n_split; s0 += BATCH) {
                    float4 dv[BATCH];
#pragma unroll
                    for (int u = 0; u < BATCH; ++u)
                        if (s0 + u < n_split) dv[u] = load4<TD>(dp + (size_t)(s0 + u) * split_stride);
#pragma unroll
                    for (int u = 0; u < BATCH; ++u)
                        if (s0 + u < n_split) { v.x += dv[u].x; v.y += dv[u].y; v.z += dv[u].z; v.w += dv[u].w; }
                }
            }
            store4(rowbuf + j, v);
            ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            float v = xr[j];
            if (delta != nullptr) {
                for (int sidx = 0; sidx < n_split; ++sidx)
                    v += to_f32(delta[(size_t)sidx * split_stride + (size_t)src * d + j]);
            }
            rowbuf[j] = v;
            ss += v * v;
        }
    }
    odin_trace_mark(2);  // loads done
    ss = block_sum(ss, red);
    odin_trace_mark(3);  // sum known
    ss /= (float)d;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    const bool write_back = (delta != nullptr) && (rows == nullptr);
    if (VEC) {
        for (int j = threadIdx.x * 4; j < d; j += blockDim.x * 4) {
            const float4 v = load4<float>(rowbuf + j);
            if (write_back) store4(xr + j, v);
            const float4 wv = (j == (int)threadIdx.x * 4) ? w0 : load4w(w, j);
            store4(o + j, make_float4(wv.x * (rs * v.x), wv.y * (rs * v.y), wv.z * (rs * v.z), wv.w * (rs * v.w)));
        }
    } else {
        for (int j = threadIdx.x; j < d; j += blockDim.x) {
            const float v = rowbuf[j];
            if (write_back) xr[j] = v;
            o[j] = from_f32<TO>(w.at(j) * (rs * v));
        }
    }
    odin_trace_mark(4);  // stores issued
}

template <typename TD, typename TO, bool VEC, int MAX_THREADS = 512>
__global__ void __launch_bounds__(MAX_THREADS, 3)
add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_split, size_t split_stride, VecRef w,
                   float eps, TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float red[32];
    extern __shared__ float rowbuf[];  // d floats
    add_rmsnorm_body<TD, TO, VEC, MAX_THREADS>(x, delta, n_split, split_stride, w, eps, out, rows, d, red, rowbuf);
}

// The variant of 1,024 threads for a few wide rows (decoding): NV groups of four per thread, kept in registers
// (no staging in shared memory), the parts' loads of a group issued together; the same order of additions as the
// kernel above, so the same bits.  Its registers are capped so that a block leaves more than a third of an SM's
// registers free: the product that follows starts its CTAs while this kernel runs, to fetch weights, and on the
// SMs that hold a row it could not (with 64 registers a thread the block took them all; those CTAs then started 4
// to 7 us after the others and the whole product ended that much later).
template <typename TD, typename TO, int NV>
__global__ void __maxnreg__(NV == 1 ? 40 : 48)
add_rmsnorm_wide_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_split, size_t split_stride, VecRef w,
                        float eps, TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    int src = r;
    if (rows != nullptr) src = rows[r];
    const int j0 = (int)threadIdx.x * 4;
    float4 w0 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j0 < d) w0 = load4w(w, j0);
    pdl_wait();
    TO* o = out + (size_t)r * d;
    if (src < 0) {
        for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = from_f32<TO>(0.f);
        return;
    }
    float* xr = x + (size_t)src * d;
    float4 v[NV];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int j = j0 + k * 4096;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < d) {
            v[k] = load4<float>(xr + j);
            if (delta != nullptr) {
                const TD* dp = delta + (size_t)src * d + j;
                for (int s0 = 0; s0 < n_split; s0 += 4) {
                    float4 dv[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (s0 + u < n_split) dv[u] = load4<TD>(dp + (size_t)(s0 + u) * split_stride);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (s0 + u < n_split) { v[k].x += dv[u].x; v[k].y += dv[u].y; v[k].z += dv[u].z; v[k].w += dv[u].w; }
                }
            }
            ss += v[k].x * v[k].x; ss += v[k].y * v[k].y; ss += v[k].z * v[k].z; ss += v[k].w * v[k].w;
        }
    }
    odin_trace_mark(2);  // loads done
    ss = block_sum(ss, red);
    odin_trace_mark(3);  // sum known
    ss /= (float)d;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    const bool write_back = (delta != nullptr) && (rows == nullptr);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int j = j0 + k * 4096;
        if (j < d) {
            if (write_back) store4(xr + j, v[k]);
            const float4 wv = (k == 0) ? w0 : load4w(w, j);
            store4(o + j, make_float4(wv.x * (rs * v[k].x), wv.y * (rs * v[k].y), wv.z * (rs * v[k].z), wv.w * (rs * v[k].w)));
        }
    }
    odin_trace_mark(4);  // stores issued
}

// Many rows (prompts), bfloat16 out: a block of 256 threads per row that keeps its NV groups of four
// per thread in registers (no staging in shared memory) and leaves room for many blocks on an SM.  With
// one 512-thread block per row and three of them per SM only 24 KB per SM were in flight, and 75 k rows
// of 2048 ran at 2.8 TB/s.  The sum of squares is added per thread over its groups in order, then over
// the block; it may differ in the last bits from the kernel above, which the 32-bit path keeps using.
template <typename TD, int NV>
__global__ void __launch_bounds__(256, NV <= 2 ? 8 : (NV <= 4 ? 5 : 3))
add_rmsnorm_rows_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_split, size_t split_stride, VecRef w,
                        float eps, bf16* __restrict__ out, int d) {
    __shared__ float red[32];
    pdl_trigger();
    const int r = blockIdx.x;
    const int nv = d / 4;
    pdl_wait();
    float* xr = x + (size_t)r * d;
    float4 v[NV];  // the norm's weights are read where they are used: all rows share them, they stay in L1
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (int)threadIdx.x + k * 256;
        if (c < nv) v[k] = load4<float>(xr + 4 * c);
    }
    if (delta != nullptr) {
        for (int s0 = 0; s0 < n_split; ++s0) {  // x, then the parts in order
            const TD* dp = delta + (size_t)s0 * split_stride + (size_t)r * d;
            float4 dv[NV];
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int c = (int)threadIdx.x + k * 256;
                if (c < nv) dv[k] = load4<TD>(dp + 4 * c);
            }
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int c = (int)threadIdx.x + k * 256;
                if (c < nv) { v[k].x += dv[k].x; v[k].y += dv[k].y; v[k].z += dv[k].z; v[k].w += dv[k].w; }
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (int)threadIdx.x + k * 256;
        if (c < nv) { ss += v[k].x * v[k].x; ss += v[k].y * v[k].y; ss += v[k].z * v[k].z; ss += v[k].w * v[k].w; }
    }
    ss = block_sum(ss, red);
    ss /= (float)d;
    ss += eps;
    const float rs = 1.0f / sqrtf(ss);
    bf16* o = out + (size_t)r * d;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = (int)threadIdx.x + k * 256;
        if (c < nv) {
            if (delta != nullptr) store4(xr + 4 * c, v[k]);
            const float4 wv = load4w(w, 4 * c);
            store4(o + 4 * c, make_float4(wv.x * (rs * v[k].x), wv.y * (rs * v[k].y), wv.z * (rs * v[k].z), wv.w * (rs * v[k].w)));
        }
    }
}

template <typename TD, int NV>
static int launch_add_rmsnorm_rows(float* x, const void* delta, int n_split, size_t split_stride, VecRef w, float eps,
                                   void* out, int n_rows, int d, cudaStream_t s) {
    odin_launch(add_rmsnorm_rows_kernel<TD, NV>, dim3(n_rows), dim3(256), 0, s, x, (const TD*)delta, n_split, split_stride, w,
                eps, (bf16*)out, d);
    ODIN_LAUNCH_CHECK();
    return 0;
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* x, const void* delta, int n_split, size_t split_stride, VecRef w,
                              float eps, void* out, const int* rows, int n_rows, int d, cudaStream_t s) {
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 200 * 1024) return ODIN_ERR_UNSUPPORTED;
    const bool vec = (d % 4 == 0) && ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)out) | ((uintptr_t)w.p)) % 16 == 0) &&
                     (split_stride % 4 == 0);
    if (vec && std::is_same<TO, bf16>::value && rows == nullptr && n_rows > 256 && d <= 8 * 256 * 4) {
        // many rows (prompts)
        if (d <= 2 * 256 * 4) return launch_add_rmsnorm_rows<TD, 2>(x, delta, n_split, split_stride, w, eps, out, n_rows, d, s);
        if (d <= 4 * 256 * 4) return launch_add_rmsnorm_rows<TD, 4>(x, delta, n_split, split_stride, w, eps, out, n_rows, d, s);
        return launch_add_rmsnorm_rows<TD, 8>(x, delta, n_split, split_stride, w, eps, out, n_rows, d, s);
    }
    if (vec) {
        // few rows (decoding): the whole row in one pass of a large block, a chain of latencies;
        // more rows: smaller blocks, more of them per SM, two passes each
        // (32-bit out: one block size per width, so that a row's sum of squares is added in the same
        // order in a prompt and in a decode step, and the 32-bit path's cuts agree bit for bit)
        // The block of 1,024 threads per row is for rows that all run at once, ahead of the few-token product.  With
        // 224 and 256 rows (two rounds of blocks, the products then on pairs of SMs) a decode step with this kernel
        // never ended under programmatic dependent launch: it ran when the kernel triggered its dependents at its end
        // instead of its start, when it was launched plainly, and with 192 rows; the cause was not found.  From 129
        // rows on the kernel of 512 threads runs, as it does for prompts.
        const bool big = !std::is_same<TO, float>::value && d >= 4096 && d <= 8192 && n_rows <= 128;
        if (big) {
            auto wide = d <= 4096 ? add_rmsnorm_wide_kernel<TD, TO, 1> : add_rmsnorm_wide_kernel<TD, TO, 2>;
            odin_launch(wide, dim3(n_rows), dim3(1024), 0, s, x, (const TD*)delta, n_split, split_stride, w, eps, (TO*)out,
                        rows, d);
            ODIN_LAUNCH_CHECK();
            return 0;
        }
        const int threads = d >= 2048 ? 512 : (d >= 1024 ? 256 : 128);
        auto kern = add_rmsnorm_kernel<TD, TO, true, 512>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        odin_launch(kern, dim3(n_rows), dim3(threads), smem, s, x, (const TD*)delta, n_split, split_stride, w, eps,
                    (TO*)out, rows, d);
    } else {
        const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        odin_launch(add_rmsnorm_kernel<TD, TO, false>, dim3(n_rows), dim3(threads), smem, s, x, (const TD*)delta, n_split,
                    split_stride, w, eps, (TO*)out, rows, d);
    }
    ODIN_LAUNCH_CHECK();
    return 0;
}

// x: [*, d] 32-bit residual stream.  delta: null, or [n_split][*, d] partial
// sums of element type delta_dtype, split_stride elements apart.  rows: null
// (row r of x -> row r of out, x updated in place), or n_rows source row
// numbers (gather; x is not written; a negative number gives a zero row).
extern "C" int odin_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_split,
                                long long split_stride, const void* w, int w_dtype, float eps, void* out,
                                int out_dtype, const int* rows, int n_rows, int d, void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    VecRef wr{w, w_dtype == ODIN_BF16};
    if (delta == nullptr) delta_dtype = ODIN_F32;
    if (delta_dtype == ODIN_F32 && out_dtype == ODIN_F32)
        return launch_add_rmsnorm<float, float>(x, delta, n_split, split_stride, wr, eps, out, rows, n_rows, d, s);
    if (delta_dtype == ODIN_F32 && out_dtype == ODIN_BF16)
        return launch_add_rmsnorm<float, bf16>(x, delta, n_split, split_stride, wr, eps, out, rows, n_rows, d, s);
    if (delta_dtype == ODIN_BF16 && out_dtype == ODIN_BF16)
        return launch_add_rmsnorm<bf16, bf16>(x, delta, n_split, split_stride, wr, eps, out, rows, n_rows, d, s);
    if (delta_dtype == ODIN_BF16 && out_dtype == ODIN_F32)
        return launch_add_rmsnorm<bf16, float>(x, delta, n_split, split_stride, wr, eps, out, rows, n_rows, d, s);
    return ODIN_ERR_UNSUPPORTED;
}

// -------------------------------------------------------------------- SwiGLU
// gu: [T, 2I], gate in columns [0, I), up in [I, 2I).  h = g * (1/(1+exp(-g))) * u
// in that order of products (infer/forward.odin:128-133).
template <typename TI, typename T>
__global__ void swiglu_kernel(const TI* __restrict__ gu, int n_split, size_t split_stride, T* __restrict__ out, int I,
                              size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int j = (int)(idx - t * I);
        float g = 0.f, u = 0.f;
        for (int s = 0; s < n_split; ++s) {
            g += to_f32(gu[(size_t)s * split_stride + t * 2 * (size_t)I + j]);
            u += to_f32(gu[(size_t)s * split_stride + t * 2 * (size_t)I + I + j]);
        }
        g *= 1.0f / (1.0f + expf(-g));
        g *= u;
        out[idx] = from_f32<T>(g);
    }
}

// The same, four columns per thread (32-bit partial sums in, bfloat16 out; I a multiple of 4, 16-byte aligned
// rows): the loads of up to four parts are in flight together.  Same order of additions and products.
__global__ void swiglu_vec_kernel(const float* __restrict__ gu, int n_split, size_t split_stride, bf16* __restrict__ out,
                                  int I, size_t total4) {
    pdl_trigger();
    pdl_wait();
    const int I4 = I / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I4;
        const int j = (int)(idx - t * I4) * 4;
        const float* row = gu + t * 2 * (size_t)I + j;
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
        for (int s0 = 0; s0 < n_split; s0 += 4) {
            float4 gv[4], uv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                if (s0 + a < n_split) {
                    gv[a] = *reinterpret_cast<const float4*>(row + (size_t)(s0 + a) * split_stride);
                    uv[a] = *reinterpret_cast<const float4*>(row + (size_t)(s0 + a) * split_stride + I);
                }
            }
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                if (s0 + a < n_split) {
                    g.x += gv[a].x; g.y += gv[a].y; g.z += gv[a].z; g.w += gv[a].w;
                    u.x += uv[a].x; u.y += uv[a].y; u.z += uv[a].z; u.w += uv[a].w;
                }
            }
        }
        g.x *= 1.0f / (1.0f + expf(-g.x)); g.x *= u.x;
        g.y *= 1.0f / (1.0f + expf(-g.y)); g.y *= u.y;
        g.z *= 1.0f / (1.0f + expf(-g.z)); g.z *= u.z;
        g.w *= 1.0f / (1.0f + expf(-g.w)); g.w *= u.w;
        store4(out + t * (size_t)I + j, g);
    }
}

// gu: [n_split][T, 2I] of in_dtype (the parts are added first), out: [T, I] of out_dtype.
extern "C" int odin_swiglu(const void* gu, int in_dtype, int n_split, long long split_stride, void* out,
                           int out_dtype, int T, int I, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = (size_t)T * I;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (in_dtype == ODIN_BF16 && out_dtype == ODIN_BF16)
        odin_launch(swiglu_kernel<bf16, bf16>, dim3((int)blocks), dim3(threads), 0, s, (const bf16*)gu, n_split,
                    (size_t)split_stride, (bf16*)out, I, total);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_F32)
        odin_launch(swiglu_kernel<float, float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, n_split,
                    (size_t)split_stride, (float*)out, I, total);
    else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16 && (I % 4) == 0 && (split_stride % 4) == 0 &&
             ((((uintptr_t)gu) | ((uintptr_t)out)) & 15) == 0) {
        size_t b4 = (total / 4 + threads - 1) / threads;
        if (b4 > 148 * 16) b4 = 148 * 16;
        odin_launch(swiglu_vec_kernel, dim3((int)b4), dim3(threads), 0, s, (const float*)gu, n_split, (size_t)split_stride,
                    (bf16*)out, I, total / 4);
    } else if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16)
        odin_launch(swiglu_kernel<float, bf16>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, n_split,
                    (size_t)split_stride, (bf16*)out, I, total);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------ random weights
// Element i of a stream is a function of (key, i) alone: two steps of splitmix64 on key + 2 i and
// key + 2 i + 1, the sum of their eight 16-bit fields, centred and scaled: a sum of eight uniforms
// computed in integers, so the host restatement (weights/random_init.py) gives the same bits.
// The product and the sum are single rounded operations (no fused multiply-add).
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean, float scale) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long h1 = mix64(key + 2ull * (unsigned long long)i);
        const unsigned long long h2 = mix64(key + 2ull * (unsigned long long)i + 1ull);
        int s = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) s += (int)((h1 >> (16 * k)) & 0xFFFFull) + (int)((h2 >> (16 * k)) & 0xFFFFull);
        const float c = (float)(s - 4 * 65535);
        out[i] = from_f32<T>(__fadd_rn(mean, __fmul_rn(c, scale)));
    }
}

extern "C" int odin_random_fill(void* out, int dtype, long long n, unsigned long long key, float mean, float scale,
                                void* stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == ODIN_F32)
        random_fill_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float*)out, n, key, mean, scale);
    else if (dtype == ODIN_BF16)
        random_fill_kernel<bf16><<<blocks, 256, 0, (cudaStream_t)stream>>>((bf16*)out, n, key, mean, scale);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------- cast
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32(in[i]));
}

extern "C" int odin_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    size_t blocks = ((size_t)n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (in_dtype == ODIN_F32 && out_dtype == ODIN_BF16)
        odin_launch(cast_kernel<float, bf16>, dim3((int)blocks), dim3(256), 0, s, (const float*)in, (bf16*)out, (size_t)n);
    else if (in_dtype == ODIN_BF16 && out_dtype == ODIN_F32)
        odin_launch(cast_kernel<bf16, float>, dim3((int)blocks), dim3(256), 0, s, (const bf16*)in, (float*)out, (size_t)n);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

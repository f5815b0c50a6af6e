// Causal grouped-query attention over the paged cache on the CUDA cores, one
// warp per (query token, query head).  It serves prompts and decoding alike in
// the 32-bit path, and is the bfloat16 path's fallback for head sizes that the
// tensor-core kernels refuse.
//
// Restates infer/forward.odin:88-115: query head h reads kv head h / (Hq/Hkv);
// score_t = (q . k_t) / sqrt(hd) for the keys t <= pos (the causal mask is the
// loop bound); softmax with the maximum subtracted (infer/ops.odin:21-37);
// out = sum_t p_t v_t.  The softmax runs "online" over chunks of 32 keys that
// start at the first visible key, so a token's result depends only on its own
// sequence and position.  A window > 0 hides keys t <= pos - window.
#include "common.cuh"
#include <math_constants.h>

#define AP_WARPS 4
#define AP_MAX_HD 512

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int hd) {
    float acc = 0.f;
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int i = 0; i < hd / 4; ++i) {
        const float4 v = k4[i];
        acc = fmaf(q[4 * i + 0], v.x, acc);
        acc = fmaf(q[4 * i + 1], v.y, acc);
        acc = fmaf(q[4 * i + 2], v.z, acc);
        acc = fmaf(q[4 * i + 3], v.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<bf16>(const float* __restrict__ q, const bf16* __restrict__ k, int hd) {
    float acc = 0.f;
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int i = 0; i < hd / 8; ++i) {
        const uint4 v = k8[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc = fmaf(q[8 * i + 2 * j], f.x, acc);
            acc = fmaf(q[8 * i + 2 * j + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(AP_WARPS * 32)
attention_plain_kernel(const T* __restrict__ q, size_t q_stride, T* __restrict__ out, size_t out_stride, int T_tok,
                       int Hq, int Hkv, int hd, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       int page_size, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ block_table, int bt_stride, int window) {
    __shared__ float qs[AP_WARPS][AP_MAX_HD];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * AP_WARPS + warp;
    if (item >= (long long)T_tok * Hq) return;
    const int t = (int)(item / Hq), h = (int)(item % Hq);
    const int seq = tok_seq[t];
    if (seq < 0) return;
    const int pos = tok_pos[t];
    const int kvh = h / (Hq / Hkv);
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
    float* qf = qs[warp];
    for (int j = lane; j < hd; j += 32) qf[j] = to_f32(qrow[j]);
    __syncwarp();

    const float inv_scale = sqrtf((float)hd);
    int t_lo = 0;
    if (window > 0 && pos - window + 1 > 0) t_lo = pos - window + 1;

    float m = -CUDART_INF_F, l = 0.f;
    float acc[AP_MAX_HD / 32];
#pragma unroll
    for (int r = 0; r < AP_MAX_HD / 32; ++r) acc[r] = 0.f;
    const int* bt = block_table + (size_t)seq * bt_stride;

    for (int t0 = t_lo; t0 <= pos; t0 += 32) {
        const int tk = t0 + lane;
        const bool valid = tk <= pos;
        long long row = -1;
        float s = -CUDART_INF_F;
        if (valid) {
            const int page = bt[tk / page_size];
            if (page >= 0) {
                row = ((long long)page * Hkv + kvh) * page_size + (tk % page_size);
                s = dot_row<T>(qf, k_cache + (size_t)row * hd, hd) / inv_scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -CUDART_INF_F) continue;  // no visible key in this chunk
        const float p = (row >= 0) ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int r = 0; r < AP_MAX_HD / 32; ++r) acc[r] *= corr;
        const int n_here = min(32, pos - t0 + 1);
        for (int j = 0; j < n_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long rj = __shfl_sync(0xffffffffu, row, j);
            if (rj < 0) continue;
            const T* vrow = v_cache + (size_t)rj * hd;
#pragma unroll
            for (int r = 0; r < AP_MAX_HD / 32; ++r) {
                const int d = r * 32 + lane;
                if (d < hd) acc[r] = fmaf(pj, to_f32(vrow[d]), acc[r]);
            }
        }
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
    const float inv_l = (l > 0.f) ? 1.0f / l : 0.f;
#pragma unroll
    for (int r = 0; r < AP_MAX_HD / 32; ++r) {
        const int d = r * 32 + lane;
        if (d < hd) orow[d] = from_f32<T>(acc[r] * inv_l);
    }
}

// q: [T, Hq*hd] with row stride q_row_stride (elements); out likewise.
extern "C" int odin_attention_plain(const void* q, long long q_row_stride, void* out, long long out_row_stride,
                                    int dtype, int T, int Hq, int Hkv, int hd, const void* k_cache,
                                    const void* v_cache, int page_size, const int* tok_pos, const int* tok_seq,
                                    const int* block_table, int bt_stride, int window, void* stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || hd > AP_MAX_HD || (hd % 8) != 0 || Hkv <= 0 || Hq % Hkv != 0) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const long long items = (long long)T * Hq;
    const long long blocks = (items + AP_WARPS - 1) / AP_WARPS;
    if (blocks > 2147483647LL) return ODIN_ERR_UNSUPPORTED;
    if (dtype == ODIN_BF16)
        odin_launch(attention_plain_kernel<bf16>, dim3((unsigned)blocks), dim3(AP_WARPS * 32), 0, s,
            (const bf16*)q, (size_t)q_row_stride, (bf16*)out, (size_t)out_row_stride, T, Hq, Hkv, hd,
            (const bf16*)k_cache, (const bf16*)v_cache, page_size, tok_pos, tok_seq, block_table, bt_stride, window);
    else if (dtype == ODIN_F32)
        odin_launch(attention_plain_kernel<float>, dim3((unsigned)blocks), dim3(AP_WARPS * 32), 0, s,
            (const float*)q, (size_t)q_row_stride, (float*)out, (size_t)out_row_stride, T, Hq, Hkv, hd,
            (const float*)k_cache, (const float*)v_cache, page_size, tok_pos, tok_seq, block_table, bt_stride,
            window);
    else
        return ODIN_ERR_UNSUPPORTED;
    ODIN_LAUNCH_CHECK();
    return 0;
}

// Per-head preparation of the fused q|k|v projection, one warp per (token, head):
//   q heads: RMSNorm over the head (optional), rotation, written to q_out (which may be
//            the projection itself: in place);
//   k heads: RMSNorm (optional), rotation, written to the paged key cache;
//   v heads: copied to the paged value cache.
// Restates infer/forward.odin:58-85 (norm before rotation, one [hd] weight shared
// by all heads, half-split pairs (i, i + rot/2)) and the cache write of :47-49.
// The rotation reads cos/sin of 32-bit angles from a table built on the host.
// All arithmetic is 32-bit.
//
// Cache layout of one layer: [page][kv head][slot in page][hd]; a sequence's
// pages are named by its row of the block table.
#include "common.cuh"
#include "head_math.cuh"

#define HP_WARPS 4
#define HP_MAX_HD 512

// TI: element type of the projection (bfloat16 or 32-bit; n_split 32-bit partial sums of a
// split product are added first, in order).  T: element type of q_out and of the cache.
template <typename TI, typename T>
__global__ void __launch_bounds__(HP_WARPS * 32)
head_prep_kernel(const TI* qkv, int n_split, size_t split_stride, T* q_out,  // may alias: no restrict
                 size_t q_out_stride, int Hq, int Hkv, int hd, size_t row_stride, VecRef qw, VecRef kw,
                 int has_norm, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                 int rot, int table_len, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                 const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_cache,
                 T* __restrict__ v_cache, int page_size, int write_kv) {
    __shared__ float buf[HP_WARPS][HP_MAX_HD];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * HP_WARPS + warp;
    const int n_heads = Hq + 2 * Hkv;
    if (head >= n_heads) return;
    const int seq = tok_seq[t];
    if (seq < 0) return;  // padding token
    const int pos = tok_pos[t];
    const TI* src = qkv + (size_t)t * row_stride + (size_t)head * hd;

    const bool is_q = head < Hq;
    const bool is_k = !is_q && head < Hq + Hkv;
    const int kvh = is_q ? 0 : (is_k ? head - Hq : head - Hq - Hkv);
    if (!is_q && !write_kv) return;

    T* dst = q_out + (size_t)t * q_out_stride + (size_t)head * hd;
    if (!is_q) {
        const int page = block_table[(size_t)seq * bt_stride + pos / page_size];
        if (page < 0) return;
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * Hkv + kvh) * page_size + (pos % page_size)) * hd;
    }

    float* b = buf[warp];
    float ss = 0.f;
    for (int j = lane; j < hd; j += 32) {
        float v = to_f32(src[j]);
        for (int sp = 1; sp < n_split; ++sp) v += to_f32(src[(size_t)sp * split_stride + j]);
        b[j] = v;
        ss += v * v;
    }
    if (!is_q && !is_k) {  // value head: stored as it is
        for (int j = lane; j < hd; j += 32) dst[j] = from_f32<T>(b[j]);
        return;
    }
    if (has_norm) {
        ss = warp_sum(ss);
        ss /= (float)hd;
        ss += eps;
        const float r = 1.0f / sqrtf(ss);
        const VecRef& w = is_q ? qw : kw;
        for (int j = lane; j < hd; j += 32) b[j] = w.at(j) * (r * b[j]);
    }
    __syncwarp();
    const int half = rot >> 1;
    const bool in_table = (pos >= 0 && pos < table_len);
    for (int j = lane; j < hd; j += 32) {
        float o;
        if (j < rot && in_table) {
            const int i = (j < half) ? j : j - half;
            const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
            const float x = b[i], y = b[i + half];
            o = (j < half) ? (x * c - y * s) : (x * s + y * c);
        } else {
            o = b[j];
        }
        dst[j] = from_f32<T>(o);
    }
}


// The common case with a bfloat16 cache (full rotary, head size 64 or 128): each lane holds
// VEC = hd/32 consecutive elements in registers, the rotation partner (i +- hd/2) lives in
// lane ^ 16, and rows move with vector loads and stores.  The input is bfloat16, or 32-bit
// partial sums of a split product that are added first, in order.  Same arithmetic as above.
using headmath::load_vec;
using headmath::store_vec_bf16;

// A warp per (token, head), TOK tokens per warp (one: for few tokens the kernel is a chain of
// latencies, and everything that can be is fetched before the wait for the kernel before it).
template <int VEC, typename TI, int TOK>
__global__ void __launch_bounds__(HP_WARPS * 32)
head_prep_fast_kernel(const TI* qkv, int n_split, size_t split_stride, bf16* q_out, size_t q_out_stride, int T, int Hq,
                      int Hkv, size_t row_stride, VecRef qw, VecRef kw, int has_norm, float eps,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ block_table, int bt_stride, bf16* __restrict__ k_cache,
                      bf16* __restrict__ v_cache, int page_size, int write_kv) {
    constexpr int HD = VEC * 32, HALF = HD / 2;
    pdl_trigger();
    // What no earlier kernel of the step writes is fetched before the wait for that kernel: the
    // step's tables, the page of the cache, the angles' cosines and sines, the norms' weights.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * HP_WARPS + warp;
    const bool in_range = head < Hq + 2 * Hkv;
    const bool is_q = head < Hq;
    const bool is_k = !is_q && head < Hq + Hkv;
    const int kvh = is_q ? 0 : (is_k ? head - Hq : head - Hq - Hkv);
    bool active[TOK], in_table[TOK];
    bf16* dst[TOK];
    float c[TOK][VEC], sn[TOK][VEC], wn[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) wn[e] = 1.f;
    if (in_range && (is_q || is_k) && has_norm) {
        const VecRef& w = is_q ? qw : kw;
#pragma unroll
        for (int e = 0; e < VEC; ++e) wn[e] = w.at(lane * VEC + e);
    }
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
        const int t = blockIdx.x * TOK + u;
        const int seq = (in_range && t < T) ? tok_seq[t] : -1;
        const int pos = (t < T) ? tok_pos[t] : 0;
        active[u] = seq >= 0 && (is_q || write_kv);
        dst[u] = q_out + (size_t)t * q_out_stride + (size_t)head * HD + lane * VEC;
        if (active[u] && !is_q) {
            const int page = block_table[(size_t)seq * bt_stride + pos / page_size];
            if (page < 0) active[u] = false;
            else dst[u] = (is_k ? k_cache : v_cache) + (((size_t)page * Hkv + kvh) * page_size + (pos % page_size)) * HD + lane * VEC;
        }
        in_table[u] = (pos >= 0 && pos < table_len);
#pragma unroll
        for (int e = 0; e < VEC; ++e) { c[u][e] = 1.f; sn[u][e] = 0.f; }
        if (active[u] && (is_q || is_k) && in_table[u]) {
            load_vec<VEC>(cos_t + (size_t)pos * HALF + (lane & 15) * VEC, c[u]);
            load_vec<VEC>(sin_t + (size_t)pos * HALF + (lane & 15) * VEC, sn[u]);
        }
    }
    pdl_wait();
    float v[TOK][VEC];
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
        if (!active[u]) continue;
        const int t = blockIdx.x * TOK + u;
        headmath::load_parts<VEC, TI>(qkv + (size_t)t * row_stride + (size_t)head * HD + lane * VEC, n_split, split_stride, v[u]);
    }
#pragma unroll
    for (int u = 0; u < TOK; ++u) {
        if (!active[u]) continue;
        if (!is_q && !is_k) {  // value head: stored as it is
            store_vec_bf16<VEC>(dst[u], v[u]);
            continue;
        }
        float o[VEC];
        headmath::norm_rotate<VEC>(v[u], has_norm != 0, wn, eps, in_table[u], c[u], sn[u], lane, o);
        store_vec_bf16<VEC>(dst[u], o);
    }
}

// For prompts: a CTA per token, its four warps share the token's heads (warp w takes heads w, w + 4,
// ...), so the angles of the token's position are fetched once per warp and not once per head, and
// four heads' loads are in flight per warp.  Same arithmetic (head_math.cuh).
template <int VEC, typename TI>
__global__ void __launch_bounds__(HP_WARPS * 32)
head_prep_token_kernel(const TI* qkv, int n_split, size_t split_stride, bf16* q_out, size_t q_out_stride, int Hq,
                       int Hkv, size_t row_stride, VecRef qw, VecRef kw, int has_norm, float eps,
                       const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len,
                       const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ block_table, int bt_stride, bf16* __restrict__ k_cache,
                       bf16* __restrict__ v_cache, int page_size, int write_kv) {
    constexpr int HD = VEC * 32, HALF = HD / 2, UNROLL = 4;
    pdl_trigger();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = tok_seq[t];
    const int pos = tok_pos[t];
    pdl_wait();
    if (seq < 0) return;
    // The first heads' loads go out before the loads that hang on the token's position (its page, its
    // angles): a CTA lives for a chain of three trips to memory otherwise, with data in flight during one.
    const int n_heads = Hq + 2 * Hkv;
    const TI* row = qkv + (size_t)t * row_stride + lane * VEC;
    float v[UNROLL][VEC];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int head = warp + u * HP_WARPS;
        if (head < n_heads && (head < Hq || write_kv))
            headmath::load_parts<VEC, TI>(row + (size_t)head * HD, n_split, split_stride, v[u]);
    }
    const int page = write_kv ? block_table[(size_t)seq * bt_stride + pos / page_size] : -1;
    const bool in_table = (pos >= 0 && pos < table_len);
    float c[VEC], sn[VEC], wq[VEC], wk[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) { c[e] = 1.f; sn[e] = 0.f; wq[e] = 1.f; wk[e] = 1.f; }
    if (in_table) {
        load_vec<VEC>(cos_t + (size_t)pos * HALF + (lane & 15) * VEC, c);
        load_vec<VEC>(sin_t + (size_t)pos * HALF + (lane & 15) * VEC, sn);
    }
    if (has_norm) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) { wq[e] = qw.at(lane * VEC + e); wk[e] = kw.at(lane * VEC + e); }
    }
    for (int h0 = warp; h0 < n_heads; h0 += HP_WARPS * UNROLL) {
        if (h0 != warp) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int head = h0 + u * HP_WARPS;
                if (head < n_heads && (head < Hq || page >= 0))
                    headmath::load_parts<VEC, TI>(row + (size_t)head * HD, n_split, split_stride, v[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int head = h0 + u * HP_WARPS;
            if (head >= n_heads) continue;
            const bool is_q = head < Hq, is_k = !is_q && head < Hq + Hkv;
            if (!is_q && page < 0) continue;
            bf16* dst;
            if (is_q) {
                dst = q_out + (size_t)t * q_out_stride + (size_t)head * HD + lane * VEC;
            } else {
                const int kvh = is_k ? head - Hq : head - Hq - Hkv;
                dst = (is_k ? k_cache : v_cache) + (((size_t)page * Hkv + kvh) * page_size + (pos % page_size)) * HD + lane * VEC;
            }
            if (!is_q && !is_k) {  // value head: stored as it is
                store_vec_bf16<VEC>(dst, v[u]);
                continue;
            }
            float o[VEC];
            headmath::norm_rotate<VEC>(v[u], has_norm != 0, is_q ? wq : wk, eps, in_table, c, sn, lane, o);
            store_vec_bf16<VEC>(dst, o);
        }
    }
}

// qkv: [n_split][T, (Hq + 2 Hkv) hd] of in_dtype (row stride row_stride, parts split_stride
// elements apart).  q_out: [T, Hq hd] of dtype (row stride q_out_stride); it may be qkv
// itself when there is one part of the same type (q is then normalised and rotated in place).
extern "C" int odin_head_prep(const void* qkv, int in_dtype, int n_split, long long split_stride, void* q_out,
                              long long q_out_stride, int dtype, int T, int Hq, int Hkv, int hd, long long row_stride,
                              const void* q_norm_w, const void* k_norm_w, int w_dtype, int has_norm, float eps,
                              const float* cos_t, const float* sin_t, int rot, int table_len,
                              const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride,
                              void* k_cache, void* v_cache, int page_size, int write_kv, void* stream) {
    if (T <= 0) return 0;
    if (hd > HP_MAX_HD || hd <= 0 || (rot & 1) || rot > hd || rot < 0 || n_split < 1) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int n_heads = Hq + 2 * Hkv;
    dim3 grid(T, (n_heads + HP_WARPS - 1) / HP_WARPS);
    if (grid.y > 65535) return ODIN_ERR_UNSUPPORTED;
    VecRef qw{q_norm_w, w_dtype == ODIN_BF16}, kw{k_norm_w, w_dtype == ODIN_BF16};
    const bool fast_in = (in_dtype == ODIN_BF16 && n_split == 1) || in_dtype == ODIN_F32;
    if (fast_in && dtype == ODIN_BF16 && rot == hd && (hd == 64 || hd == 128) && (row_stride % 4) == 0 &&
        (split_stride % 4) == 0 && (q_out_stride % 4) == 0 &&
        ((((uintptr_t)qkv) | ((uintptr_t)q_out) | ((uintptr_t)cos_t) | ((uintptr_t)sin_t)) & 15) == 0) {
#define FAST(VEC, TI, TOK)                                                                                         \
    odin_launch(head_prep_fast_kernel<VEC, TI, TOK>, dim3((T + TOK - 1) / TOK, grid.y), dim3(HP_WARPS * 32), 0, s,     \
                (const TI*)qkv, n_split, (size_t)split_stride, (bf16*)q_out, (size_t)q_out_stride, T, Hq, Hkv,         \
                (size_t)row_stride, qw, kw, has_norm, eps, cos_t, sin_t, table_len, tok_pos, tok_seq, block_table,      \
                bt_stride, (bf16*)k_cache, (bf16*)v_cache, page_size, write_kv)
#define FAST_T(VEC, TI)                                                                                            \
    do {                                                                                                           \
        if (T >= 256)                                                                                              \
            odin_launch(head_prep_token_kernel<VEC, TI>, dim3(T), dim3(HP_WARPS * 32), 0, s, (const TI*)qkv, n_split,  \
                        (size_t)split_stride, (bf16*)q_out, (size_t)q_out_stride, Hq, Hkv, (size_t)row_stride, qw, kw, \
                        has_norm, eps, cos_t, sin_t, table_len, tok_pos, tok_seq, block_table, bt_stride,              \
                        (bf16*)k_cache, (bf16*)v_cache, page_size, write_kv);                                           \
        else FAST(VEC, TI, 1);                                                                                     \
    } while (0)
        if (hd == 128 && in_dtype == ODIN_BF16) FAST_T(4, bf16);
        else if (hd == 128) FAST_T(4, float);
        else if (in_dtype == ODIN_BF16) FAST_T(2, bf16);
        else FAST_T(2, float);
#undef FAST_T
#undef FAST
        ODIN_LAUNCH_CHECK();
        return 0;
    }
#define GO(TI, TT)                                                                                                  \
    odin_launch(head_prep_kernel<TI, TT>, grid, dim3(HP_WARPS * 32), 0, s,                                           \
        (const TI*)qkv, n_split, (size_t)split_stride, (TT*)q_out, (size_t)q_out_stride, Hq, Hkv, hd,               \
        (size_t)row_stride, qw, kw, has_norm, eps, cos_t, sin_t, rot, table_len, tok_pos, tok_seq, block_table,     \
        (int)bt_stride, (TT*)k_cache, (TT*)v_cache, page_size, write_kv)
    if (in_dtype == ODIN_BF16 && dtype == ODIN_BF16) GO(bf16, bf16);
    else if (in_dtype == ODIN_F32 && dtype == ODIN_F32) GO(float, float);
    else if (in_dtype == ODIN_F32 && dtype == ODIN_BF16) GO(float, bf16);
    else return ODIN_ERR_UNSUPPORTED;
#undef GO
    ODIN_LAUNCH_CHECK();
    return 0;
}

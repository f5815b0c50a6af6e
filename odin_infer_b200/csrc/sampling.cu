// Sampling over rows of 32-bit logits, one thread block per sequence.
//
// Restates sampler/sampler.odin on the device:
//   argmax: the first maximum wins (strict >, :79-89);
//   temperature: logits / T, softmax with the maximum subtracted, one coin in
//     [0,1) per token, walk of the cumulative sum in index order (:91-100, :179-185);
//   top-p: keep the most probable tokens until their sum first exceeds topp, scale the
//     coin by that sum and walk the kept ones in order of falling probability (:106-139);
//   repetition penalty: each distinct recent token has a positive logit divided
//     and a negative one multiplied (:143-160).
// The logits are never modified by the sampling kernels (the reference
// overwrites the caller's logits with probabilities; this does not).
// All sums run in an order fixed by the block size, so a seed gives the same
// tokens whatever else is in the batch.
#include "common.cuh"
#include <math_constants.h>

#define SB 1024  // threads per block

// ------------------------------------------------------------------ argmax
__global__ void __launch_bounds__(SB) argmax_kernel(const float* __restrict__ logits, size_t ld, int V,
                                                    int* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SB) {
        const float v = row[i];
        if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
    }
    // NaN-free logits assumed; ties go to the lower index.
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = sv[lane];
        bi = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
}

extern "C" int odin_argmax(const float* logits, long long ld, int B, int V, int* out, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0) return ODIN_ERR_BAD_ARG;
    odin_launch(argmax_kernel, dim3(B), dim3(SB), 0, (cudaStream_t)stream, logits, (size_t)ld, V, out);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------- temperature / top-p draw
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = red[lane];  // SB = 1024 threads = 32 warps
    return warp_max(t);
}

// Sum of e_i = exp(l_i / T - m) over the tokens with e_i >= thr.
__device__ __forceinline__ float masked_sum(const float* row, int V, float inv_t, float m, float thr, float* red) {
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += SB) {
        const float e = expf(row[i] * inv_t - m);
        if (e >= thr) s += e;
    }
    return block_sum(s, red);
}

// The largest t in [lo, hi] (bit patterns of positive floats, which order like the floats) with
// S(t) = sum of e_i >= t  >  target, given S(lo) > target.  S falls as t grows.  Eight probes per
// pass over the row, so 2^30 candidates take ten passes instead of thirty.
__device__ unsigned search_threshold(const float* row, int V, float inv_t, float m, float target, unsigned lo,
                                     unsigned hi, float* red) {
    constexpr int P = 8;
    while (lo < hi) {
        const unsigned span = hi - lo;  // probes lo < p_0 < ... <= hi
        unsigned probe[P];
        float acc[P];
#pragma unroll
        for (int q = 0; q < P; ++q) {
            probe[q] = lo + (unsigned)(((unsigned long long)span * (q + 1) + P - 1) / P);
            acc[q] = 0.f;
        }
        for (int i = threadIdx.x; i < V; i += SB) {
            const float e = expf(row[i] * inv_t - m);
#pragma unroll
            for (int q = 0; q < P; ++q)
                if (e >= __uint_as_float(probe[q])) acc[q] += e;
        }
        int best = -1;
#pragma unroll
        for (int q = 0; q < P; ++q) {
            const float sq = block_sum(acc[q], red);
            if (sq > target) best = q;  // S is monotone: the last probe that still exceeds the target
        }
        if (best < 0) hi = probe[0] - 1;
        else {
            if (best + 1 < P) hi = probe[best + 1] - 1;
            lo = probe[best];
        }
    }
    return lo;
}

// Temperature draw.  Without top-p: the cumulative sum is walked in index order (sample_mult,
// sampler/sampler.odin:91-100).  With 0 < top_p < 1 the reference sorts the candidates by falling
// probability, cuts after the first whose cumulative sum exceeds topp, scales the coin by that sum and
// walks the sorted list (sample_topp, :106-139).  Here nothing is sorted: the token at which a walk in
// falling order crosses a mark r is the one with the largest value u such that the tokens of at least
// that value sum to more than r, which a search over u finds (ties: in index order).  So the same coin
// gives the reference's token, up to the rounding of the sums and the order among exactly equal
// probabilities, which the reference's unstable sort leaves open.
__global__ void __launch_bounds__(SB) sample_kernel(const float* __restrict__ logits, size_t ld, int V,
                                                    float temperature, float top_p,
                                                    const float* __restrict__ coins, int* __restrict__ out) {
    __shared__ float red[32];
    __shared__ float chunk_sum[SB];
    __shared__ int chosen;
    pdl_trigger();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    const float inv_t = 1.0f / temperature;
    float mx = -CUDART_INF_F;
    for (int i = threadIdx.x; i < V; i += SB) mx = fmaxf(mx, row[i] * inv_t);
    mx = block_max(mx, red);
    const float total = masked_sum(row, V, inv_t, mx, 0.f, red);
    const int per = (V + SB - 1) / SB;  // contiguous chunk of the row per thread, for walks in index order
    const int c0 = min(V, (int)threadIdx.x * per), c1 = min(V, c0 + per);
    if (threadIdx.x == 0) chosen = -1;

    if (top_p > 0.f && top_p < 1.f && V > 1) {
        // everything in units of e (unnormalised probabilities)
        const float cutoff = (1.0f - top_p) / (float)(V - 1) * total;
        const float target = top_p * total;
        const float s_cut = masked_sum(row, V, inv_t, mx, cutoff, red);
        unsigned lo = __float_as_uint(fmaxf(cutoff, 1e-45f));
        float cumulative = s_cut;  // the candidates together do not exceed topp: all of them stay
        if (s_cut > target) {
            // v: the value of the candidate at which the cumulative sum first exceeds topp
            lo = search_threshold(row, V, inv_t, mx, target, lo, __float_as_uint(1.0f), red);
            const float v = __uint_as_float(lo);
            const float above = masked_sum(row, V, inv_t, mx, __uint_as_float(lo + 1), red);
            const float ties = floorf((target - above) / v) + 1.0f;  // how many of value v it takes
            cumulative = above + fmaxf(ties, 1.0f) * v;
        }
        const float r = coins[blockIdx.x] * cumulative;
        unsigned ub = lo;
        float u = __uint_as_float(lo);
        int nth = 0x7fffffff;  // which of the tokens of value u, in index order (beyond their number: the last)
        if (masked_sum(row, V, inv_t, mx, u, red) > r) {
            ub = search_threshold(row, V, inv_t, mx, r, lo, __float_as_uint(1.0f), red);
            u = __uint_as_float(ub);
            const float above = masked_sum(row, V, inv_t, mx, __uint_as_float(ub + 1), red);
            nth = (int)fminf(floorf(fmaxf(r - above, 0.f) / u), 2.0e9f);
        }
        // the nth token (from 0) whose e is exactly u, else the last such one; if u is below every
        // candidate (the coin scaled to the whole sum), the smallest candidate's last occurrence
        float cnt = 0.f;
        for (int i = c0; i < c1; ++i) cnt += (expf(row[i] * inv_t - mx) == u) ? 1.f : 0.f;
        chunk_sum[threadIdx.x] = cnt;
        __syncthreads();
        if (threadIdx.x == 0) {
            int seen = 0, owner = -1, last_owner = -1;
            for (int t = 0; t < SB; ++t) {
                const int c = (int)chunk_sum[t];
                if (c > 0) last_owner = t;
                if (owner < 0 && seen + c > nth) { owner = t; break; }
                seen += c;
            }
            if (owner < 0) { owner = last_owner; seen = 0x7fffffff; }
            if (owner >= 0) {
                const int o0 = min(V, owner * per), o1 = min(V, o0 + per);
                int pick = -1;
                for (int i = o0; i < o1; ++i) {
                    if (expf(row[i] * inv_t - mx) == u) {
                        pick = i;
                        if (seen != 0x7fffffff && seen++ == nth) break;
                    }
                }
                chosen = pick;
            }
        }
        __syncthreads();
        if (chosen < 0) {
            // no token of value u (u was the cutoff itself): the smallest candidate, the reference's last_idx
            float best = CUDART_INF_F;
            for (int i = threadIdx.x; i < V; i += SB) {
                const float e = expf(row[i] * inv_t - mx);
                if (e >= u) best = fminf(best, e);
            }
            best = -block_max(-best, red);
            int last = -1;
            for (int i = threadIdx.x; i < V; i += SB)
                if (expf(row[i] * inv_t - mx) == best) last = max(last, i);
            const float lf = block_max((float)last, red);
            if (threadIdx.x == 0) chosen = (int)lf;
            __syncthreads();
        }
        if (threadIdx.x == 0) out[blockIdx.x] = max(chosen, 0);
        return;
    }

    // ---- all tokens, cumulative walk in index order: contiguous chunk per thread, then a scan
    const float target = coins[blockIdx.x] * total;
    float cs = 0.f;
    for (int i = c0; i < c1; ++i) cs += expf(row[i] * inv_t - mx);
    chunk_sum[threadIdx.x] = cs;
    __syncthreads();
    if (threadIdx.x == 0) {
        // serial exclusive scan over 1024 chunk sums: fixed order
        float run = 0.f;
        int owner = -1;
        for (int t = 0; t < SB; ++t) {
            const float nxt = run + chunk_sum[t];
            if (target < nxt) { owner = t; break; }
            run = nxt;
        }
        if (owner >= 0) {
            const int o0 = min(V, owner * per), o1 = min(V, o0 + per);
            float cdf = run;
            int pick = -1;
            for (int i = o0; i < o1; ++i) {
                cdf += expf(row[i] * inv_t - mx);
                if (target < cdf) { pick = i; break; }
            }
            chosen = (pick >= 0) ? pick : o1 - 1;
        }
    }
    __syncthreads();
    // rounding left the coin beyond the last sum: the last token (reference: n - 1)
    if (threadIdx.x == 0) out[blockIdx.x] = (chosen >= 0) ? chosen : V - 1;
}

extern "C" int odin_sample(const float* logits, long long ld, int B, int V, float temperature, float top_p,
                           const float* coins, int* out, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !(temperature > 0.f)) return ODIN_ERR_BAD_ARG;
    odin_launch(sample_kernel, dim3(B), dim3(SB), 0, (cudaStream_t)stream, logits, (size_t)ld, V, temperature, top_p, coins, out);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------ repetition penalty
// recent: [B, W] token ids, negative = empty.  logits are changed in place (the
// caller passes a copy).
__global__ void repetition_penalty_kernel(float* __restrict__ logits, size_t ld, int V,
                                          const int* __restrict__ recent, int W, float penalty) {
    pdl_trigger();
    pdl_wait();
    float* row = logits + (size_t)blockIdx.x * ld;
    const int* rec = recent + (size_t)blockIdx.x * W;
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        const int tok = rec[j];
        if (tok < 0 || tok >= V) continue;
        bool dup = false;
        for (int i = 0; i < j; ++i) dup |= (rec[i] == tok);
        if (dup) continue;
        const float v = row[tok];
        row[tok] = (v > 0.f) ? v / penalty : v * penalty;
    }
}

extern "C" int odin_repetition_penalty(float* logits, long long ld, int B, int V, const int* recent, int W,
                                       float penalty, void* stream) {
    if (B <= 0 || W <= 0) return 0;
    odin_launch(repetition_penalty_kernel, dim3(B), dim3(128), 0, (cudaStream_t)stream, logits, (size_t)ld, V, recent, W, penalty);
    ODIN_LAUNCH_CHECK();
    return 0;
}

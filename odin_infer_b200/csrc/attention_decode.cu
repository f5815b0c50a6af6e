// Attention of one new token per sequence over its paged bfloat16 cache, split
// along the keys so that a small batch still occupies every SM.
//
// Two kernels.  The general one (any head size that is a power of two from 16 to 256), on the
// CUDA cores: grid (key splits, kv heads x query-head groups, sequences); a CTA takes one
// sequence, one kv head, up to G of its query heads, and a contiguous range of the
// sequence's pages; every key and value it loads serves all G query heads.  Inside
// a warp a key's head_dim elements are spread over LPK lanes (16-byte loads, whole
// rows coalesced), so one warp instruction covers 32/LPK keys.  Each lane group
// keeps an "online softmax" of its own (running maximum, sum, weighted values);
// groups, warps and finally splits are merged with the usual rescaling, the splits by a
// second kernel.  The tensor-core one (head sizes 64 and 128; further down): pages by TMA,
// both products on mma.sync, the splits merged inside the kernel, optionally with head
// preparation inside.
//
// Arithmetic follows infer/forward.odin:88-115 (scores scaled by 1/sqrt(hd), softmax
// with the maximum subtracted, weighted sum of values), all in 32-bit; the scale and
// log2(e) are folded into q so that the exponentials are exp2.
//
// Scratch: partial results [sequence][query head][split] of head_dim + 2 floats, in
// memory the caller provides.
#include "attn_common.cuh"
#include "head_math.cuh"
#include <math_constants.h>

#include <type_traits>

namespace {

constexpr int AD_WARPS = 4;
constexpr float NEG_BIG = -1.0e30f;

template <int HD>
struct Geo {
    static constexpr int EPL = (HD >= 64) ? 16 : 8;  // elements per lane
    static constexpr int LPK = HD / EPL;             // lanes per key
    static constexpr int KPI = 32 / LPK;             // keys per warp instruction
    static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must give a power-of-two lane count");
};

template <int N>
__device__ __forceinline__ void load_bf16(const bf16* p, float (&out)[N]) {
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
        const uint4 v = reinterpret_cast<const uint4*>(p)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            out[8 * i + 2 * j] = f.x;
            out[8 * i + 2 * j + 1] = f.y;
        }
    }
}

template <int HD, int G>
__global__ void __launch_bounds__(AD_WARPS * 32)
attn_decode_kernel(const bf16* __restrict__ q, size_t q_stride, int Hq, int Hkv, const bf16* __restrict__ k_cache,
                   const bf16* __restrict__ v_cache, int page_size, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_seq, const int* __restrict__ block_table, int bt_stride, int window,
                   float scale_log2, float* __restrict__ part_acc, float* __restrict__ part_ml, int n_split) {
    using GE = Geo<HD>;
    constexpr int EPL = GE::EPL, LPK = GE::LPK, KPI = GE::KPI;
    pdl_trigger();
    pdl_wait();
    const int split = blockIdx.x;
    const int g_total = Hq / Hkv;
    const int g_parts = (g_total + G - 1) / G;
    const int kvh = blockIdx.y / g_parts;
    const int h0 = kvh * g_total + (blockIdx.y % g_parts) * G;   // first query head of this CTA
    const int n_h = min(G, kvh * g_total + g_total - h0);
    const int t = blockIdx.z;                                    // token row = sequence of the step
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPK, kg = lane / LPK;

    const int seq = tok_seq[t];
    float* my_acc = part_acc + (((size_t)t * Hq + h0) * n_split + split) * HD;
    float* my_ml = part_ml + (((size_t)t * Hq + h0) * n_split + split) * 2;
    const size_t head_step_acc = (size_t)n_split * HD, head_step_ml = (size_t)n_split * 2;

    int t_lo = 0, t_hi = 0;  // keys [t_lo, t_hi) of this split
    if (seq >= 0) {
        const int pos = tok_pos[t];
        int first = 0;
        if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;
        const int p_first = first / page_size, p_last = pos / page_size;
        const int n_pages = p_last - p_first + 1;
        const int per = (n_pages + n_split - 1) / n_split;
        const int pa = p_first + split * per, pb = min(p_last + 1, pa + per);
        t_lo = max(first, pa * page_size);
        t_hi = min(pos + 1, pb * page_size);
    }

    float qf[G][EPL], acc[G][EPL], m[G], l[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = NEG_BIG;
        l[h] = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) { acc[h][e] = 0.f; qf[h][e] = 0.f; }
        if (h < n_h && seq >= 0) {
            load_bf16<EPL>(q + (size_t)t * q_stride + (size_t)(h0 + h) * HD + sub * EPL, qf[h]);
#pragma unroll
            for (int e = 0; e < EPL; ++e) qf[h][e] *= scale_log2;
        }
    }

    // the page numbers of this split, once, so that the loop's loads do not wait for them
    constexpr int PG_CAP = 128;
    __shared__ int s_pg[PG_CAP];
    const int* bt = block_table + (size_t)max(seq, 0) * bt_stride;
    const int pg0 = t_lo / page_size;
    const int n_pg = (t_hi > t_lo) ? ((t_hi - 1) / page_size - pg0 + 1) : 0;
    for (int i = threadIdx.x; i < min(n_pg, PG_CAP); i += AD_WARPS * 32) s_pg[i] = bt[pg0 + i];
    __syncthreads();

    auto key_row = [&](int tk, size_t& row) -> bool {
        if (tk >= t_hi) return false;
        const int pi = tk / page_size - pg0;
        const int page = (pi < PG_CAP) ? s_pg[pi] : bt[pg0 + pi];
        if (page < 0) return false;
        row = (((size_t)page * Hkv + kvh) * page_size + (tk % page_size)) * HD + sub * EPL;
        return true;
    };
    auto absorb = [&](bool have, const float (&kf)[EPL], const float (&vf)[EPL]) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) s = fmaf(qf[h][e], kf[e], s);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (have) {
                const float m_new = fmaxf(m[h], s);
                const float corr = exp2f(m[h] - m_new);
                const float p = exp2f(s - m_new);
                l[h] = l[h] * corr + p;
#pragma unroll
                for (int e = 0; e < EPL; ++e) acc[h][e] = fmaf(p, vf[e], acc[h][e] * corr);
                m[h] = m_new;
            }
        }
    };
    // two batches of keys per trip, all four loads issued before the arithmetic
    for (int base = t_lo + warp * KPI; base < t_hi; base += 2 * AD_WARPS * KPI) {
        float k0[EPL], v0[EPL], k1[EPL], v1[EPL];
        size_t r0 = 0, r1 = 0;
        const bool h0v = key_row(base + kg, r0);
        const bool h1v = key_row(base + AD_WARPS * KPI + kg, r1);
        if (h0v) { load_bf16<EPL>(k_cache + r0, k0); load_bf16<EPL>(v_cache + r0, v0); }
        if (h1v) { load_bf16<EPL>(k_cache + r1, k1); load_bf16<EPL>(v_cache + r1, v1); }
        if (!h0v) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) { k0[e] = 0.f; v0[e] = 0.f; }
        }
        if (!h1v) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) { k1[e] = 0.f; v1[e] = 0.f; }
        }
        absorb(h0v, k0, v0);
        if (base + AD_WARPS * KPI < t_hi) absorb(h1v, k1, v1);
    }

    // merge the lane groups of the warp (lanes that hold the same elements of different keys)
#pragma unroll
    for (int h = 0; h < G; ++h) {
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float m_o = __shfl_xor_sync(0xffffffffu, m[h], o);
            const float l_o = __shfl_xor_sync(0xffffffffu, l[h], o);
            const float m_new = fmaxf(m[h], m_o);
            const float ca = exp2f(m[h] - m_new), cb = exp2f(m_o - m_new);
            l[h] = l[h] * ca + l_o * cb;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float a_o = __shfl_xor_sync(0xffffffffu, acc[h][e], o);
                acc[h][e] = acc[h][e] * ca + a_o * cb;
            }
            m[h] = m_new;
        }
    }

    // merge the warps through shared memory
    __shared__ float s_acc[AD_WARPS][G][HD];
    __shared__ float s_ml[AD_WARPS][G][2];
    if (kg == 0) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) s_acc[warp][h][sub * EPL + e] = acc[h][e];
            if (sub == 0) { s_ml[warp][h][0] = m[h]; s_ml[warp][h][1] = l[h]; }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += AD_WARPS * 32) {
        const int h = idx / HD, d = idx % HD;
        if (h >= n_h) continue;
        float mm = s_ml[0][h][0];
#pragma unroll
        for (int w = 1; w < AD_WARPS; ++w) mm = fmaxf(mm, s_ml[w][h][0]);
        float a = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float c = exp2f(s_ml[w][h][0] - mm);
            a += s_acc[w][h][d] * c;
            ll += s_ml[w][h][1] * c;
        }
        my_acc[(size_t)h * head_step_acc + d] = a;
        if (d == 0) {
            my_ml[(size_t)h * head_step_ml] = mm;
            my_ml[(size_t)h * head_step_ml + 1] = ll;
        }
    }
}

// ---------------------------------------------------------------------------
// The tensor-core variant (head sizes 64 and 128, up to 16 query heads per kv head).
//
// A CTA of 4 warps takes (sequence, kv head, key split).  The query heads of the kv
// head are the rows of a 16-row MMA tile.  The split's pages stream through a ring of
// SLOTS shared-memory slots by TMA (one page of one kv head is a contiguous [64, hd]
// tile; 128-byte swizzle).  Page i of the split belongs to warp i mod 4, which computes
// S = Q K^T and O += P V for its 64 keys with mma.sync m16n8k16 and keeps its own
// running maximum and sum; when it is done with a page it asks for the page that uses
// the slot next.  No warp waits for another inside the loop: with a few pages per CTA
// the kernel is a chain of latencies, and four pages are in flight per CTA instead of
// a quarter of one per warp.  The four warps' results are merged through shared
// memory at the end, then either written as this split's partial or, with one split,
// normalised and stored as the result.
// ---------------------------------------------------------------------------
struct DecodeTcParams {
    const bf16* q;
    size_t q_stride;
    bf16* out;
    size_t out_stride;
    int Hq, Hkv;
    const int* tok_pos;
    const int* tok_seq;
    const int* block_table;
    int bt_stride;
    int window;
    float scale_log2;
    float* part_acc;
    float* part_ml;
    int n_split;
    int* error;
    int* counters;  // one per (token, kv head), zero between launches: how many splits have written their partial
    // With head preparation inside the kernel (PREP): q, k and v come from the fused projection's
    // output, [n_parts][tokens, (Hq + 2 Hkv) hd] partial sums; the new key and value go to the cache.
    const void* qkv;
    size_t qkv_row_stride, qkv_part_stride;
    int qkv_parts;
    VecRef q_norm, k_norm;
    int has_norm;
    float eps;
    const float* cos_t;
    const float* sin_t;
    int table_len;
    bf16* k_cache;
    bf16* v_cache;
    int write_kv;
};

// The splits of one (token, kv head) meet here once their partials are written: the one that
// arrives last adds them up, writes the result and leaves the counter at zero for the next
// launch.  out[h][:] = sum_s w_s acc_s / sum_s w_s l_s with w_s = 2^(m_s - max m).
template <int HD>
__device__ __forceinline__ void split_arrive_and_combine(const DecodeTcParams& p, int t, int kvh, int g, int h0,
                                                         int* s_last) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *s_last = (atomicAdd(&p.counters[t * p.Hkv + kvh], 1) == p.n_split - 1);
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    for (int idx = threadIdx.x * 4; idx < g * HD; idx += 128 * 4) {
        const int r = idx / HD, d = idx % HD;
        const float* ml = p.part_ml + ((size_t)t * p.Hq + h0 + r) * p.n_split * 2;
        const float* ac = p.part_acc + ((size_t)t * p.Hq + h0 + r) * p.n_split * HD + d;
        float mm = NEG_BIG;
        for (int s0 = 0; s0 < p.n_split; ++s0) mm = fmaxf(mm, __ldcg(ml + 2 * s0));
        float ll = 0.f;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < p.n_split; s0 += 4) {
            float4 v[4];
            float w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (s0 + u < p.n_split) {
                    v[u] = __ldcg(reinterpret_cast<const float4*>(ac + (size_t)(s0 + u) * HD));
                    w[u] = exp2f(__ldcg(ml + 2 * (s0 + u)) - mm);
                    ll += __ldcg(ml + 2 * (s0 + u) + 1) * w[u];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (s0 + u < p.n_split) {
                    a.x += v[u].x * w[u]; a.y += v[u].y * w[u]; a.z += v[u].z * w[u]; a.w += v[u].w * w[u];
                }
            }
        }
        const float inv = ll > 0.f ? 1.0f / ll : 0.f;
        uint2 u2;
        u2.x = attn::pack_bf16(a.x * inv, a.y * inv);
        u2.y = attn::pack_bf16(a.z * inv, a.w * inv);
        *reinterpret_cast<uint2*>(p.out + (size_t)t * p.out_stride + (size_t)(h0 + r) * HD + d) = u2;
    }
    if (threadIdx.x == 0) p.counters[t * p.Hkv + kvh] = 0;
}

__device__ __forceinline__ uint32_t q_off(int row, int col) {  // a [16 x HD] tile in 64-column sub-tiles of 2 KB
    const int sub = col >> 6, chunk = (col & 63) >> 3;
    return (uint32_t)(sub * 2048 + row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <int HD, int SLOTS>
struct DecodeTcSmem {
    static constexpr int TILE = attn::PAGE_T * HD * 2;  // K or V of one page
    static constexpr int SLOT = 2 * TILE;
    static constexpr int BT_KEEP = 128;
    static constexpr int OS = HD + 8;                   // row of the merge buffer (floats), padded against bank conflicts
    static constexpr int TAIL = 16 * HD * 2 /*Q*/ + 64 /*barriers, flag*/ + 4 * 16 * 2 * 4 /*m, l*/ + 4 * 16 * 4 /*scales*/ +
                                BT_KEEP * 4 + 32 /*requests per slot*/;
    static constexpr int BYTES = SLOTS * SLOT + TAIL + 1024 /*alignment*/;
    static_assert(4 * 16 * OS * 4 <= SLOTS * SLOT, "the merge buffer reuses the page slots");
    static_assert(SLOTS <= 7, "barriers and the flag share 64 bytes");
};

// PREP 0: q is given and the cache is complete.  PREP 1 (32-bit parts) and 2 (bfloat16): the
// kernel prepares its own heads (per-head RMSNorm and rotation, as head_prep.cu does): every
// CTA its query heads, and the CTA whose pages include the newest one that token's key and
// value, which it writes to the cache and into its own copy of the page.  The kernel before it
// is then the projection itself, and every page can be requested before that one is done.
template <int HD, int SLOTS, int PREP>
__global__ void __launch_bounds__(128)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const DecodeTcParams p) {
    using namespace attn;
    using TI = typename std::conditional<PREP == 2, bf16, float>::type;
    constexpr int VEC = HD / 32;
    using L = DecodeTcSmem<HD, SLOTS>;
    constexpr int TILE = L::TILE, SLOT = L::SLOT, BT_KEEP = L::BT_KEEP, OS = L::OS;
    constexpr int KB = HD / 16, NB_O = HD / 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem + SLOTS * SLOT;  // 16 x HD
    uint64_t* full = reinterpret_cast<uint64_t*>(sQ + 16 * HD * 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(full + 7);
    int* s_last = const_cast<int*>(abort_flag) + 1;
    float* s_ml = reinterpret_cast<float*>(full + 8);  // [4 warps][16 rows][2]
    float* s_scale = s_ml + 4 * 16 * 2;                // [4 warps][16 rows]
    int* s_pages = reinterpret_cast<int*>(s_scale + 4 * 16);
    volatile int* s_requested = s_pages + BT_KEEP;     // [SLOTS] how many pages have been requested into the slot

    const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();
    // The step's tables are written before the step starts, and of the cache the kernel before
    // this one writes only the newest key and value (in the last page): tables and the older
    // pages are fetched before the wait for that kernel, the query and the last page after it.
    const int seq = p.tok_seq[t];
    if (seq < 0) { pdl_wait(); return; }  // padding row
    const int g = p.Hq / p.Hkv, h0 = kvh * g;
    const int pos = p.tok_pos[t];
    int first = 0;
    if (p.window > 0 && pos - p.window + 1 > 0) first = pos - p.window + 1;
    const int p_first = first / PAGE_T, p_last = pos / PAGE_T;
    const int per = (p_last - p_first + 1 + p.n_split - 1) / p.n_split;
    const int pa = p_first + split * per, pb = min(p_last + 1, pa + per);  // pages [pa, pb)
    const int n_here = pb - pa;
    const int t_lo = first, t_hi = pos + 1;                               // visible keys [t_lo, t_hi)
    float* my_acc = p.part_acc + (((size_t)t * p.Hq + h0) * p.n_split + split) * HD;
    float* my_ml = p.part_ml + (((size_t)t * p.Hq + h0) * p.n_split + split) * 2;
    const size_t head_step_acc = (size_t)p.n_split * HD, head_step_ml = (size_t)p.n_split * 2;
    if (n_here <= 0) {  // nothing for this split: an empty partial
        pdl_wait();
        for (int idx = threadIdx.x; idx < g * HD; idx += 128) {
            const int r = idx / HD, d = idx % HD;
            my_acc[(size_t)r * head_step_acc + d] = 0.f;
            if (d == 0) { my_ml[(size_t)r * head_step_ml] = NEG_BIG; my_ml[(size_t)r * head_step_ml + 1] = 0.f; }
        }
        split_arrive_and_combine<HD>(p, t, kvh, g, h0, s_last);
        return;
    }
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;

    // this CTA's page numbers, so that no trip to the block table sits between two pages
    for (int i = threadIdx.x; i < min(n_here, BT_KEEP); i += 128) s_pages[i] = bt[pa + i];
    auto issue = [&](int i, int slot) {  // page pa + i of the sequence into a slot
        const int page = (i < BT_KEEP) ? s_pages[i] : bt[pa + i];
        const int row = (page * p.Hkv + kvh) * PAGE_T;
        uint8_t* dst = smem + slot * SLOT;
        tc::mbar_expect_tx(&full[slot], SLOT);
#pragma unroll
        for (int sub = 0; sub < HD / 64; ++sub) {
            tc::tma_load_2d(dst + sub * 8192, &map_k, sub * 64, row, &full[slot]);
            tc::tma_load_2d(dst + TILE + sub * 8192, &map_v, sub * 64, row, &full[slot]);
        }
        __threadfence_block();
        s_requested[slot] = i / SLOTS + 1;
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < SLOTS; ++s) { tc::mbar_init(&full[s], 1); s_requested[s] = 0; }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int i = 0; i < SLOTS && i < n_here; ++i)
            if (PREP != 0 || pa + i != p_last) issue(i, i);
    float new_k[VEC], new_v[VEC];  // PREP: the newest key and value, in the warp that takes the last page
    const bool has_last = (p_last >= pa && p_last < pb);
    const int last_warp = (p_last - pa) & 3;
    if (PREP == 0) {
        pdl_wait();
        for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += 128) {
            const int r = idx / (HD / 8), c = idx % (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < g) v = *reinterpret_cast<const uint4*>(p.q + (size_t)t * p.q_stride + (size_t)(h0 + r) * HD + c * 8);
            *reinterpret_cast<uint4*>(sQ + q_off(r, c * 8)) = v;
        }
        if (threadIdx.x == 0 && has_last && p_last - pa < SLOTS) issue(p_last - pa, p_last - pa);
    } else {
        // before the wait: constants of this token's position and the norms' weights
        const bool in_table = (pos >= 0 && pos < p.table_len);
        float c[VEC], sn[VEC], wq[VEC], wk[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { c[e] = 1.f; sn[e] = 0.f; wq[e] = 1.f; wk[e] = 1.f; }
        if (in_table) {
            headmath::load_vec<VEC>(p.cos_t + (size_t)pos * (HD / 2) + (lane & 15) * VEC, c);
            headmath::load_vec<VEC>(p.sin_t + (size_t)pos * (HD / 2) + (lane & 15) * VEC, sn);
        }
        if (p.has_norm) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) { wq[e] = p.q_norm.at(lane * VEC + e); wk[e] = p.k_norm.at(lane * VEC + e); }
        }
        for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += 128)
            *reinterpret_cast<uint4*>(sQ + idx * 16) = make_uint4(0, 0, 0, 0);
        __syncthreads();
        pdl_wait();
        const TI* row = reinterpret_cast<const TI*>(p.qkv) + (size_t)t * p.qkv_row_stride + lane * VEC;
        for (int r = warp; r < g; r += 4) {
            float v[VEC], o[VEC];
            headmath::load_parts<VEC, TI>(row + (size_t)(h0 + r) * HD, p.qkv_parts, p.qkv_part_stride, v);
            headmath::norm_rotate<VEC>(v, p.has_norm != 0, wq, p.eps, in_table, c, sn, lane, o);
            headmath::store_vec_bf16<VEC>(reinterpret_cast<bf16*>(sQ + q_off(r, lane * VEC)) + ((lane * VEC) & 7), o);
        }
        if (has_last && warp == last_warp) {
            float v[VEC];
            headmath::load_parts<VEC, TI>(row + (size_t)(p.Hq + kvh) * HD, p.qkv_parts, p.qkv_part_stride, v);
            headmath::norm_rotate<VEC>(v, p.has_norm != 0, wk, p.eps, in_table, c, sn, lane, new_k);
            headmath::load_parts<VEC, TI>(row + (size_t)(p.Hq + p.Hkv + kvh) * HD, p.qkv_parts, p.qkv_part_stride, new_v);
        }
    }
    __syncthreads();

    uint32_t qa[KB][4];
    const uint32_t sQ_u = tc::smem_u32(sQ);
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) ldmatrix_x4(qa[kb], sQ_u + q_off(lane & 15, kb * 16 + (lane >> 4) * 8));

    float o[NB_O][4];
#pragma unroll
    for (int i = 0; i < NB_O; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};

    for (int i = warp; i < n_here; i += 4) {
        const int slot = i % SLOTS, pg = pa + i;
        const uint32_t phase = (i / SLOTS) & 1;
        // A wait by parity cannot tell the slot's use before this one from the one that has not
        // begun: the warp first waits until its page has been requested (by the warp that had the
        // slot before, or at the start), only then for the page to land.
        bool ok = true;
        if (s_requested[slot] <= i / SLOTS) {
            unsigned long long t0 = 0;
            for (uint32_t n = 1; s_requested[slot] <= i / SLOTS; ++n) {
                if (*abort_flag) { ok = false; break; }
                if ((n & 255) == 0) {
                    const unsigned long long now = tc::global_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > TC_WAIT_SECONDS * 1000000000ull) { *abort_flag = 1; ok = false; break; }
                }
            }
        }
        ok = ok && tc::mbar_wait(&full[slot], phase, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) break;
        uint8_t* sK = smem + slot * SLOT;
        uint8_t* sV = sK + TILE;
        const uint32_t sK_u = tc::smem_u32(sK), sV_u = tc::smem_u32(sV);
        if (PREP != 0 && pg == p_last) {
            // the newest key and value: into this CTA's copy of the page, and into the cache
            const int rrow = pos % PAGE_T;
            headmath::store_vec_bf16<VEC>(reinterpret_cast<bf16*>(sK + tile_off(rrow, lane * VEC)), new_k);
            headmath::store_vec_bf16<VEC>(reinterpret_cast<bf16*>(sV + tile_off(rrow, lane * VEC)), new_v);
            if (p.write_kv) {
                const int page = (i < BT_KEEP) ? s_pages[i] : bt[pa + i];
                const size_t at = (((size_t)page * p.Hkv + kvh) * PAGE_T + rrow) * HD + lane * VEC;
                headmath::store_vec_bf16<VEC>(p.k_cache + at, new_k);
                headmath::store_vec_bf16<VEC>(p.v_cache + at, new_v);
            }
            __syncwarp();
        }
        if (pg == p_last) {
            // slots past the sequence's end may hold a stale Inf or NaN; 0 x NaN is NaN: clear those value rows
            const int valid = t_hi - pg * PAGE_T;
            if (valid < PAGE_T) {
                for (int idx = lane; idx < (PAGE_T - valid) * (HD / 8); idx += 32) {
                    const int r = valid + idx / (HD / 8), c = idx % (HD / 8);
                    *reinterpret_cast<uint4*>(sV + tile_off(r, c * 8)) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
        }
        // S = Q K^T for the page's 64 keys: eight blocks of eight keys
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[nb][j] = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, sK_u + tile_off(np * 16 + (lane & 7) + ((lane >> 4) << 3), kb * 16 + ((lane >> 3) & 1) * 8));
                mma_bf16(s[2 * np], qa[kb], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qa[kb], b[2], b[3]);
            }
        }
        const int key0 = pg * PAGE_T + (lane & 3) * 2;
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tk = key0 + nb * 8 + (j & 1);
                float v = s[nb][j] * p.scale_log2;
                if (tk < t_lo || tk >= t_hi) v = -CUDART_INF_F;
                s[nb][j] = v;
                mx[j >> 1] = fmaxf(mx[j >> 1], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            m_use[r] = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            corr[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float pv = exp2f(s[nb][j] - m_use[j >> 1]);
                s[nb][j] = pv;
                l_run[j >> 1] += pv;
            }
        }
#pragma unroll
        for (int n = 0; n < NB_O; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        // O += P V, sixteen keys at a time
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t pf[4];
            pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int nb2 = 0; nb2 < NB_O / 2; ++nb2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, sV_u + tile_off(ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), nb2 * 16 + (lane >> 4) * 8));
                mma_bf16(o[2 * nb2], pf, b[0], b[1]);
                mma_bf16(o[2 * nb2 + 1], pf, b[2], b[3]);
            }
        }
        __syncwarp();  // every lane is done with the slot
        if (lane == 0 && i + SLOTS < n_here) issue(i + SLOTS, slot);
    }
    __syncthreads();  // no warp reads a slot any more and every requested page has been consumed
    if (*abort_flag) {
        if (threadIdx.x == 0 && p.error != nullptr) atomicExch(p.error, 1);
        return;
    }

    // merge the four warps (each saw its own pages) through shared memory
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    float* s_o = reinterpret_cast<float*>(smem);  // [4 warps][16 rows][OS]
    const int row_a = lane >> 2, col = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < NB_O; ++n) {
        float* dst = s_o + ((size_t)warp * 16 + row_a) * OS + n * 8 + col;
        *reinterpret_cast<float2*>(dst) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(dst + 8 * OS) = make_float2(o[n][2], o[n][3]);
    }
    if ((lane & 3) == 0) {
        s_ml[(warp * 16 + row_a) * 2] = fmaxf(m_run[0], NEG_BIG);
        s_ml[(warp * 16 + row_a) * 2 + 1] = l_run[0];
        s_ml[(warp * 16 + row_a + 8) * 2] = fmaxf(m_run[1], NEG_BIG);
        s_ml[(warp * 16 + row_a + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    if (threadIdx.x < 64) {  // each warp's weight in each row
        const int r = threadIdx.x & 15, w = threadIdx.x >> 4;
        float mm = NEG_BIG;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) mm = fmaxf(mm, s_ml[(w2 * 16 + r) * 2]);
        s_scale[w * 16 + r] = exp2f(s_ml[(w * 16 + r) * 2] - mm);
    }
    __syncthreads();
    for (int idx = threadIdx.x * 4; idx < g * HD; idx += 128 * 4) {
        const int r = idx / HD, d = idx % HD;  // four consecutive columns of one row
        float mm = NEG_BIG, ll = 0.f;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float c = s_scale[w * 16 + r];
            const float4 v = *reinterpret_cast<const float4*>(s_o + ((size_t)w * 16 + r) * OS + d);
            a.x += v.x * c; a.y += v.y * c; a.z += v.z * c; a.w += v.w * c;
            ll += s_ml[(w * 16 + r) * 2 + 1] * c;
            mm = fmaxf(mm, s_ml[(w * 16 + r) * 2]);
        }
        if (p.n_split == 1) {
            const float inv = ll > 0.f ? 1.0f / ll : 0.f;
            uint2 u;
            u.x = pack_bf16(a.x * inv, a.y * inv);
            u.y = pack_bf16(a.z * inv, a.w * inv);
            *reinterpret_cast<uint2*>(p.out + (size_t)t * p.out_stride + (size_t)(h0 + r) * HD + d) = u;
        } else {
            *reinterpret_cast<float4*>(my_acc + (size_t)r * head_step_acc + d) = a;
            if (d == 0) { my_ml[(size_t)r * head_step_ml] = mm; my_ml[(size_t)r * head_step_ml + 1] = ll; }
        }
    }
    if (p.n_split > 1) split_arrive_and_combine<HD>(p, t, kvh, g, h0, s_last);
}

// out[t][h][:] = sum_s w_s acc_s / sum_s w_s l_s, w_s = 2^(m_s - max m)
__global__ void attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int n_split,
                                    int hd, bf16* __restrict__ out, size_t out_stride, int Hq,
                                    const int* __restrict__ tok_seq) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x / Hq, h = blockIdx.x % Hq;
    if (tok_seq[t] < 0) return;
    const float* ml = part_ml + ((size_t)t * Hq + h) * n_split * 2;
    const float* ac = part_acc + ((size_t)t * Hq + h) * n_split * hd;
    float mm = NEG_BIG;
    for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, ml[2 * s]);
    float ll = 0.f;
    for (int s = 0; s < n_split; ++s) ll += ml[2 * s + 1] * exp2f(ml[2 * s] - mm);
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < n_split; ++s) a += ac[(size_t)s * hd + d] * exp2f(ml[2 * s] - mm);
        out[(size_t)t * out_stride + (size_t)h * hd + d] = __float2bfloat16_rn(a * inv);
    }
}

template <int HD>
int launch_decode(const bf16* q, size_t q_stride, bf16* out, size_t out_stride, int B, int Hq, int Hkv,
                  const bf16* k_cache, const bf16* v_cache, int page_size, const int* tok_pos, const int* tok_seq,
                  const int* block_table, int bt_stride, int window, float* part_acc, float* part_ml, int n_split,
                  cudaStream_t s) {
    const int g = Hq / Hkv;
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
#define GO(G)                                                                                                      \
    do {                                                                                                           \
        dim3 grid(n_split, Hkv * ((g + G - 1) / G), B);                                                            \
        odin_launch(attn_decode_kernel<HD, G>, grid, dim3(AD_WARPS * 32), 0, s, q, q_stride, Hq, Hkv, k_cache,      \
                    v_cache, page_size, tok_pos, tok_seq, block_table, bt_stride, window, scale_log2, part_acc,    \
                    part_ml, n_split);                                                                             \
    } while (0)
    if (g == 1) GO(1);
    else if (g == 2) GO(2);
    else if (g == 3) GO(3);
    else GO(4);
#undef GO
    ODIN_LAUNCH_CHECK();
    odin_launch(attn_combine_kernel, dim3(B * Hq), dim3(HD < 128 ? 32 : 128), 0, s, (const float*)part_acc,
                (const float*)part_ml, n_split, (int)HD, out, out_stride, Hq, tok_seq);
    ODIN_LAUNCH_CHECK();
    return 0;
}


// The error flag and the split counters live in the library's device image, so that no entry
// point of this file ever allocates device memory.  In host code these names are only handles
// for cudaGetSymbolAddress.
constexpr int SPLIT_COUNTERS = 1 << 16;
static __device__ int g_decode_error;
static __device__ int g_split_counters[SPLIT_COUNTERS];

template <typename T>
int* device_symbol(const T& symbol) {
    constexpr int MAX_DEVICES = 64;
    static int* addr[MAX_DEVICES] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> g(mu);
    if (addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, symbol) != cudaSuccess) return nullptr;
        addr[dev] = static_cast<int*>(p);
    }
    return addr[dev];
}

int* decode_error_flag() { return device_symbol(g_decode_error); }
int* split_counters() { return device_symbol(g_split_counters); }

template <int HD, int SLOTS, int PREP>
int launch_decode_tc_slots(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTcParams& p, dim3 grid, cudaStream_t s) {
    constexpr int SMEM = DecodeTcSmem<HD, SLOTS>::BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_kernel<HD, SLOTS, PREP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    odin_launch(attn_decode_tc_kernel<HD, SLOTS, PREP>, grid, dim3(128), (size_t)SMEM, s, mk, mv, p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// What head preparation inside the kernel needs (see DecodeTcParams).
struct PrepArgs {
    const void* qkv;
    int in_dtype, parts;
    size_t row_stride, part_stride;
    VecRef q_norm, k_norm;
    int has_norm;
    float eps;
    const float* cos_t;
    const float* sin_t;
    int table_len;
    int write_kv;
};

template <int HD>
int launch_decode_tc(const bf16* q, size_t q_stride, bf16* out, size_t out_stride, int B, int Hq, int Hkv,
                     const bf16* k_cache, const bf16* v_cache, int n_pages, const int* tok_pos, const int* tok_seq,
                     const int* block_table, int bt_stride, int window, float* part_acc, float* part_ml, int n_split,
                     cudaStream_t s, const PrepArgs* prep = nullptr) {
    // the result is written with 8-byte stores
    if ((out_stride % 4) != 0 || (((uintptr_t)out) & 7) != 0) return ODIN_ERR_UNSUPPORTED;
    CUtensorMap mk, mv;
    int rc;
    const long long rows = (long long)n_pages * Hkv * attn::PAGE_T;
    if ((rc = attn::cache_map(&mk, k_cache, rows, HD))) return rc;
    if ((rc = attn::cache_map(&mv, v_cache, rows, HD))) return rc;
    DecodeTcParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
    p.Hq = Hq; p.Hkv = Hkv; p.tok_pos = tok_pos; p.tok_seq = tok_seq;
    p.block_table = block_table; p.bt_stride = bt_stride; p.window = window;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    p.part_acc = part_acc; p.part_ml = part_ml; p.n_split = n_split;
    p.error = decode_error_flag();
    p.counters = split_counters();
    if (n_split > 1 && (p.counters == nullptr || (long long)B * Hkv > SPLIT_COUNTERS)) return ODIN_ERR_UNSUPPORTED;
    int mode = 0;
    if (prep != nullptr) {
        p.qkv = prep->qkv; p.qkv_row_stride = prep->row_stride; p.qkv_part_stride = prep->part_stride;
        p.qkv_parts = prep->parts; p.q_norm = prep->q_norm; p.k_norm = prep->k_norm; p.has_norm = prep->has_norm;
        p.eps = prep->eps; p.cos_t = prep->cos_t; p.sin_t = prep->sin_t; p.table_len = prep->table_len;
        p.k_cache = const_cast<bf16*>(k_cache); p.v_cache = const_cast<bf16*>(v_cache); p.write_kv = prep->write_kv;
        mode = prep->in_dtype == ODIN_F32 ? 1 : 2;
    }
    dim3 grid(n_split, Hkv, B);
    // few CTAs: one per SM with a deep ring; many: two per SM with a ring half as deep
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const long long ctas = (long long)n_split * Hkv * B;
    const bool deep = ctas <= sms;
#define GO(PREP)                                                                  \
    (deep ? launch_decode_tc_slots<HD, 6, PREP>(mk, mv, p, grid, s)               \
          : launch_decode_tc_slots<HD, 3, PREP>(mk, mv, p, grid, s))
    if (mode == 0) return GO(0);
    if (mode == 1) return GO(1);
    return GO(2);
#undef GO
}

}  // namespace

// Floats of scratch that odin_attention_decode needs for B tokens, Hq query heads and n_split key splits.
extern "C" long long odin_attention_decode_scratch(int B, int Hq, int hd, int n_split) {
    return (long long)B * Hq * n_split * (hd + 2);
}

extern "C" int odin_attention_decode_error() {
    int* f = decode_error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) {
        cudaMemset(f, 0, sizeof(int));
        // splits of the failed launch may never have met: their counters start from zero again
        if (int* c = split_counters()) cudaMemset(c, 0, SPLIT_COUNTERS * sizeof(int));
    }
    return v;
}

// Does the split kernel take this head size?  (Others go to the plain kernel.)
extern "C" int odin_attention_decode_supported(int hd) {
    return hd == 16 || hd == 32 || hd == 64 || hd == 128 || hd == 256;
}

// One query token per row of q ([B, Hq*hd] bfloat16, row stride q_row_stride); row t
// belongs to sequence tok_seq[t] (row of the block table; negative: padding, skipped)
// at position tok_pos[t].  n_pages: pages of the cache line (0: unknown, the tensor-core
// kernel is then not used).  scratch: odin_attention_decode_scratch(...) floats.
extern "C" int odin_attention_decode(const void* q, long long q_row_stride, void* out, long long out_row_stride, int B,
                                     int Hq, int Hkv, int hd, const void* k_cache, const void* v_cache, int page_size,
                                     int n_pages, const int* tok_pos, const int* tok_seq, const int* block_table,
                                     int bt_stride, int window, float* scratch, int n_split, void* stream) {
    if (B <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0 || n_split < 1 || scratch == nullptr) return ODIN_ERR_BAD_ARG;
    if (B > 65535 || Hq > 65535 || n_split > 65535) return ODIN_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)B * Hq * n_split * hd;
    // head sizes 64 and 128 with at most 16 query heads per kv head: the tensor-core kernel
    if ((hd == 64 || hd == 128) && Hq / Hkv <= 16 && page_size == attn::PAGE_T && n_pages > 0 &&
        (q_row_stride % 8) == 0 && (((uintptr_t)q) & 15) == 0 && (out_row_stride % 4) == 0 &&
        (((uintptr_t)out) & 7) == 0 && (((uintptr_t)scratch) & 15) == 0) {
        if (hd == 64)
            return launch_decode_tc<64>((const bf16*)q, (size_t)q_row_stride, (bf16*)out, (size_t)out_row_stride, B, Hq,
                                        Hkv, (const bf16*)k_cache, (const bf16*)v_cache, n_pages, tok_pos, tok_seq,
                                        block_table, bt_stride, window, part_acc, part_ml, n_split, s);
        return launch_decode_tc<128>((const bf16*)q, (size_t)q_row_stride, (bf16*)out, (size_t)out_row_stride, B, Hq,
                                     Hkv, (const bf16*)k_cache, (const bf16*)v_cache, n_pages, tok_pos, tok_seq,
                                     block_table, bt_stride, window, part_acc, part_ml, n_split, s);
    }
#define CALL(HD)                                                                                                  \
    return launch_decode<HD>((const bf16*)q, (size_t)q_row_stride, (bf16*)out, (size_t)out_row_stride, B, Hq, Hkv, \
                             (const bf16*)k_cache, (const bf16*)v_cache, page_size, tok_pos, tok_seq, block_table, \
                             bt_stride, window, part_acc, part_ml, n_split, s)
    switch (hd) {
        case 16: CALL(16);
        case 32: CALL(32);
        case 64: CALL(64);
        case 128: CALL(128);
        case 256: CALL(256);
        default: return ODIN_ERR_UNSUPPORTED;
    }
#undef CALL
}

// Decode attention that prepares its own heads: qkv is the fused projection's output for the
// step's B tokens, [parts][B, (Hq + 2 Hkv) hd] of in_dtype (32-bit partial sums, parts
// part_stride elements apart, or one bfloat16 part); q and k get their per-head RMSNorm
// (has_norm) and the rotation by the position's angles (cos_t, sin_t: [table_len, hd/2]);
// the new key and value are written to the cache (write_kv) and attended to.  The same
// arithmetic as odin_head_prep followed by odin_attention_decode, in one kernel.  Refuses
// (ODIN_ERR_UNSUPPORTED) what the tensor-core kernel does not take; the caller then runs the two.
extern "C" int odin_attention_decode_fused(const void* qkv, int in_dtype, int parts, long long part_stride,
                                           long long row_stride, void* out, long long out_row_stride, int B, int Hq,
                                           int Hkv, int hd, const void* q_norm_w, const void* k_norm_w, int w_dtype,
                                           int has_norm, float eps, const float* cos_t, const float* sin_t, int rot,
                                           int table_len, void* k_cache, void* v_cache, int page_size, int n_pages,
                                           const int* tok_pos, const int* tok_seq, const int* block_table,
                                           int bt_stride, int window, float* scratch, int n_split, int write_kv,
                                           void* stream) {
    if (B <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0 || n_split < 1 || scratch == nullptr || parts < 1) return ODIN_ERR_BAD_ARG;
    if (B > 65535 || Hq > 65535 || n_split > 65535) return ODIN_ERR_UNSUPPORTED;
    const bool in_ok = (in_dtype == ODIN_F32) || (in_dtype == ODIN_BF16 && parts == 1);
    if (!((hd == 64 || hd == 128) && rot == hd && Hq / Hkv <= 16 && page_size == attn::PAGE_T && n_pages > 0 && in_ok &&
          (row_stride % 4) == 0 && (part_stride % 4) == 0 && (out_row_stride % 4) == 0 &&
          ((((uintptr_t)qkv) | ((uintptr_t)cos_t) | ((uintptr_t)sin_t) | ((uintptr_t)scratch)) & 15) == 0 &&
          (((uintptr_t)out) & 7) == 0))
        return ODIN_ERR_UNSUPPORTED;
    PrepArgs prep;
    prep.qkv = qkv; prep.in_dtype = in_dtype; prep.parts = parts;
    prep.row_stride = (size_t)row_stride; prep.part_stride = (size_t)part_stride;
    prep.q_norm = VecRef{q_norm_w, w_dtype == ODIN_BF16};
    prep.k_norm = VecRef{k_norm_w, w_dtype == ODIN_BF16};
    prep.has_norm = has_norm; prep.eps = eps; prep.cos_t = cos_t; prep.sin_t = sin_t; prep.table_len = table_len;
    prep.write_kv = write_kv;
    cudaStream_t s = (cudaStream_t)stream;
    float* part_acc = scratch;
    float* part_ml = scratch + (size_t)B * Hq * n_split * hd;
    if (hd == 64)
        return launch_decode_tc<64>(nullptr, 0, (bf16*)out, (size_t)out_row_stride, B, Hq, Hkv, (const bf16*)k_cache,
                                    (const bf16*)v_cache, n_pages, tok_pos, tok_seq, block_table, bt_stride, window,
                                    part_acc, part_ml, n_split, s, &prep);
    return launch_decode_tc<128>(nullptr, 0, (bf16*)out, (size_t)out_row_stride, B, Hq, Hkv, (const bf16*)k_cache,
                                 (const bf16*)v_cache, n_pages, tok_pos, tok_seq, block_table, bt_stride, window,
                                 part_acc, part_ml, n_split, s, &prep);
}

// ---------------------------------------------------------------------------
// The variant that allocates nothing (see attention_decode_noalloc.h).
// ---------------------------------------------------------------------------
#include <mutex>

#include "attention_decode_noalloc.h"

// The scratch of the no-allocation entry point.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_scratch[ODIN_NOALLOC_SCRATCH_FLOATS];

extern "C" long long odin_attention_decode_noalloc_need(int B, int Hq, int hd, int n_split) {
    return odin_attention_decode_scratch(B, Hq, hd, n_split);
}

extern "C" int odin_attention_decode_noalloc(const void* q, long long q_row_stride, void* out, long long out_row_stride,
                                             int B, int Hq, int Hkv, int hd, const void* k_cache, const void* v_cache,
                                             int page_size, int n_pages, const int* tok_pos, const int* tok_seq,
                                             const int* block_table, int bt_stride, int window, int n_split,
                                             void* stream) {
    if (B <= 0) return 0;
    if (Hq <= 0 || hd <= 0 || n_split < 1) return ODIN_ERR_BAD_ARG;
    if (odin_attention_decode_scratch(B, Hq, hd, n_split) > (long long)ODIN_NOALLOC_SCRATCH_FLOATS)
        return ODIN_ERR_TOO_LARGE;
    // once per device, with that device current: the array's address on this device
    constexpr int MAX_DEVICES = 64;
    static float* addr[MAX_DEVICES] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return ODIN_ERR_UNSUPPORTED;
    float* scratch;
    {
        std::lock_guard<std::mutex> g(mu);
        if (addr[dev] == nullptr) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess) return (int)e;
            addr[dev] = static_cast<float*>(p);
        }
        scratch = addr[dev];
    }
    return odin_attention_decode(q, q_row_stride, out, out_row_stride, B, Hq, Hkv, hd, k_cache, v_cache, page_size,
                                 n_pages, tok_pos, tok_seq, block_table, bt_stride, window, scratch, n_split, stream);
}

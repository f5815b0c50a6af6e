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
#include "attention_decode_tc.cuh"

namespace {

constexpr int AD_WARPS = 4;
using attn_decode::NEG_BIG;

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
using attn_decode::DecodeTcParams;
using attn_decode::DecodeTcSmem;

// The kernel of its own: a CTA of four warps per (key split, kv head, sequence).
template <int HD, int SLOTS, int PREP>
__global__ void __launch_bounds__(128)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const DecodeTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    pdl_trigger();
    attn_decode::attn_decode_tc_body<HD, SLOTS, PREP, 0>(map_k, map_v, p, smem, (int)threadIdx.x, (int)blockIdx.x,
                                                         (int)blockIdx.y, (int)blockIdx.z, [] { pdl_wait(); });
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
    // very few CTAs: a deep ring each; else a ring half as deep, with which a CTA fits an SM beside the CTA of the
    // projection before it (and a second one of its own kind) and has its pages before that projection is done
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    const long long ctas = (long long)n_split * Hkv * B;
    static int deep_upto = -1;
    if (deep_upto < 0) { const char* e = getenv("ODIN_DECODE_DEEP_UPTO"); deep_upto = e ? atoi(e) : 32; }
    const bool deep = ctas <= deep_upto;
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

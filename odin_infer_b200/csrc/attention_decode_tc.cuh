// Decode attention on the tensor cores for one (sequence, kv head, key split): the parameters, the
// meeting of the key splits and the body of the kernel, shared by the kernel of its own
// (attention_decode.cu) and by kernels that run it as one of their phases.
#pragma once

#include <math_constants.h>

#include <type_traits>

#include "attn_common.cuh"
#include "head_math.cuh"

namespace attn_decode {

constexpr float NEG_BIG = -1.0e30f;

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
// The 128 threads of a group meet (see attn_decode_tc_body).
template <int BAR>
__device__ __forceinline__ void group_sync() {
    asm volatile("bar.sync %0, 128;" ::"n"(BAR) : "memory");
}

template <int HD, int BAR>
__device__ __forceinline__ void split_arrive_and_combine(const DecodeTcParams& p, int t, int kvh, int g, int h0,
                                                         int* s_last, const int tid) {
    __threadfence();
    group_sync<BAR>();
    if (tid == 0) *s_last = (atomicAdd(&p.counters[t * p.Hkv + kvh], 1) == p.n_split - 1);
    group_sync<BAR>();
    if (!*s_last) return;
    __threadfence();
    for (int idx = tid * 4; idx < g * HD; idx += 128 * 4) {
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
    if (tid == 0) p.counters[t * p.Hkv + kvh] = 0;
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

// One page (64 keys) of one warp's online softmax: S = Q K^T, the running maximum and sum, O += P V.
// sK_u, sV_u: the page's key and value tiles in shared memory (tile_off layout); qa: the warp's query
// fragments (16 rows x HD); keys outside [t_lo, t_hi) are masked; page_key0: position of the page's first key.
template <int HD>
__device__ __forceinline__ void attend_page(const uint32_t sK_u, const uint32_t sV_u, const uint32_t (&qa)[HD / 16][4],
                                            float (&o)[HD / 8][4], float (&m_run)[2], float (&l_run)[2],
                                            const int page_key0, const int t_lo, const int t_hi, const float scale_log2,
                                            const int lane) {
    using namespace attn;
    constexpr int KB = HD / 16, NB_O = HD / 8;
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
    const int key0 = page_key0 + (lane & 3) * 2;
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tk = key0 + nb * 8 + (j & 1);
            float v = s[nb][j] * scale_log2;
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
}

// PREP 0: q is given and the cache is complete.  PREP 1 (32-bit parts) and 2 (bfloat16): the
// kernel prepares its own heads (per-head RMSNorm and rotation, as head_prep.cu does): every
// CTA its query heads, and the CTA whose pages include the newest one that token's key and
// value, which it writes to the cache and into its own copy of the page.  The kernel before it
// is then the projection itself, and every page can be requested before that one is done.
// The kernel's body for a group of 128 threads (tid 0..127) that meet on named barrier BAR: a whole CTA
// (BAR 0: the CTA's own barrier) or four warps of a larger one.  smem: DecodeTcSmem<HD, SLOTS>::BYTES - 1024
// bytes, 1024-byte aligned.  (split, kvh, t): which piece of the work.  wait_before(): called by all 128
// threads together, once, where the body first needs what ran before it (the stand-alone kernel waits for
// the kernel before it there); tables, weights and the cache's older pages are read ahead of it.
template <int HD, int SLOTS, int PREP, int BAR, typename WaitFn>
__device__ __forceinline__ void attn_decode_tc_body(const CUtensorMap& map_k, const CUtensorMap& map_v,
                                                    const DecodeTcParams& p, uint8_t* smem, const int tid,
                                                    const int split, const int kvh, const int t, WaitFn&& wait_before) {
    using namespace attn;
    using TI = typename std::conditional<PREP == 2, bf16, float>::type;
    constexpr int VEC = HD / 32;
    using L = DecodeTcSmem<HD, SLOTS>;
    constexpr int TILE = L::TILE, SLOT = L::SLOT, BT_KEEP = L::BT_KEEP, OS = L::OS;
    constexpr int KB = HD / 16, NB_O = HD / 8;
    uint8_t* sQ = smem + SLOTS * SLOT;  // 16 x HD
    uint64_t* full = reinterpret_cast<uint64_t*>(sQ + 16 * HD * 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(full + 7);
    int* s_last = const_cast<int*>(abort_flag) + 1;
    float* s_ml = reinterpret_cast<float*>(full + 8);  // [4 warps][16 rows][2]
    float* s_scale = s_ml + 4 * 16 * 2;                // [4 warps][16 rows]
    int* s_pages = reinterpret_cast<int*>(s_scale + 4 * 16);
    volatile int* s_requested = s_pages + BT_KEEP;     // [SLOTS] how many pages have been requested into the slot

    const int warp = tid >> 5, lane = tid & 31;
    // The step's tables are written before the step starts, and of the cache the kernel before
    // this one writes only the newest key and value (in the last page): tables and the older
    // pages are fetched before the wait for that kernel, the query and the last page after it.
    const int seq = p.tok_seq[t];
    if (seq < 0) { wait_before(); return; }  // padding row
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
        wait_before();
        for (int idx = tid; idx < g * HD; idx += 128) {
            const int r = idx / HD, d = idx % HD;
            my_acc[(size_t)r * head_step_acc + d] = 0.f;
            if (d == 0) { my_ml[(size_t)r * head_step_ml] = NEG_BIG; my_ml[(size_t)r * head_step_ml + 1] = 0.f; }
        }
        split_arrive_and_combine<HD, BAR>(p, t, kvh, g, h0, s_last, tid);
        return;
    }
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;

    // this CTA's page numbers, so that no trip to the block table sits between two pages
    for (int i = tid; i < min(n_here, BT_KEEP); i += 128) s_pages[i] = bt[pa + i];
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
    if (tid == 0) {
        for (int s = 0; s < SLOTS; ++s) { tc::mbar_init(&full[s], 1); s_requested[s] = 0; }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    group_sync<BAR>();
    if (tid == 0)
        for (int i = 0; i < SLOTS && i < n_here; ++i)
            if (PREP != 0 || pa + i != p_last) issue(i, i);
    float new_k[VEC], new_v[VEC];  // PREP: the newest key and value, in the warp that takes the last page
    const bool has_last = (p_last >= pa && p_last < pb);
    const int last_warp = (p_last - pa) & 3;
    if (PREP == 0) {
        wait_before();
        for (int idx = tid; idx < 16 * (HD / 8); idx += 128) {
            const int r = idx / (HD / 8), c = idx % (HD / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < g) v = *reinterpret_cast<const uint4*>(p.q + (size_t)t * p.q_stride + (size_t)(h0 + r) * HD + c * 8);
            *reinterpret_cast<uint4*>(sQ + q_off(r, c * 8)) = v;
        }
        if (tid == 0 && has_last && p_last - pa < SLOTS) issue(p_last - pa, p_last - pa);
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
        for (int idx = tid; idx < 16 * (HD / 8); idx += 128)
            *reinterpret_cast<uint4*>(sQ + idx * 16) = make_uint4(0, 0, 0, 0);
        group_sync<BAR>();
        wait_before();
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
    group_sync<BAR>();
    odin_trace_mark(2);  // the query heads are prepared

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
        attend_page<HD>(sK_u, sV_u, qa, o, m_run, l_run, pg * PAGE_T, t_lo, t_hi, p.scale_log2, lane);
        __syncwarp();  // every lane is done with the slot
        if (lane == 0 && i + SLOTS < n_here) issue(i + SLOTS, slot);
    }
    group_sync<BAR>();  // no warp reads a slot any more and every requested page has been consumed
    odin_trace_mark(3);  // every page is multiplied
    if (*abort_flag) {
        if (tid == 0 && p.error != nullptr) atomicExch(p.error, 1);
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
    group_sync<BAR>();
    if (tid < 64) {  // each warp's weight in each row
        const int r = tid & 15, w = tid >> 4;
        float mm = NEG_BIG;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) mm = fmaxf(mm, s_ml[(w2 * 16 + r) * 2]);
        s_scale[w * 16 + r] = exp2f(s_ml[(w * 16 + r) * 2] - mm);
    }
    group_sync<BAR>();
    for (int idx = tid * 4; idx < g * HD; idx += 128 * 4) {
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
    odin_trace_mark(4);  // the warps are merged, the result or the partial is written
    if (p.n_split > 1) split_arrive_and_combine<HD, BAR>(p, t, kvh, g, h0, s_last, tid);
    odin_trace_mark(5);  // the splits have met
}


}  // namespace attn_decode

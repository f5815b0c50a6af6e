// Causal grouped-query attention of prompts on the 5th-generation tensor cores.
//
// A CTA of 320 threads takes 128 consecutive query tokens of one sequence and one
// query head and walks over the sequence's cache pages (64 keys each):
//   warp 0      TMA producer: K and V page tiles, two stages each; K page j and V page j - 2 arrive under
//               one barrier, because the MMA thread needs both at the same point of its program;
//   warp 1      allocates tensor memory and issues the MMAs (one thread):
//               S = Q K^T (tcgen05.mma M128 N64, K and Q both K-major), then
//               O += P V (M128 N=head_dim, P read from tensor memory, V MN-major exactly
//               as the cache stores it), accumulators S and O in TMEM; one commit per page (behind the
//               scores after next) tells the softmax, the next rescaling and the producer (stages free);
//   warps 2..9  two threads per query row (32 keys of the page each; the row maximum is
//               exchanged through shared memory): read S from TMEM, mask, online
//               softmax in 32-bit registers (exponentials as ex2 of one fused
//               multiply-add), write P as packed bfloat16 back into the columns of the S
//               buffer just read, rescale O in TMEM only when the row maximum ran ahead
//               of the scaling maximum by more than 2^8, and at the end normalise and store.
// S has two buffers in TMEM, so the scores of the next page are computed while the softmax of the
// current one runs; two CTAs share an SM (96 KB of shared memory and 256 TMEM columns each) and fill
// each other's gaps.  The CTAs are persistent and walk the (head, sequence, tile) triples back and forth.
//
// Measured on one CTA with clock marks (2,048 tokens, head size 128): a page costs ~1,900 cycles.  The MMA
// thread issues for ~1,500 of them and waits ~400 for P; a softmax thread works ~1,450 and waits the rest for
// scores.  Per S buffer the chain "P handed over, P V and the scores after next issued, softmax" is serial (the
// next scores overwrite P), so a page costs about the larger of the two plus the two hand-overs; the tensor core
// itself would need 570 cycles per page and SM (measured in isolation, mma_probe.cu: an MMA of N 64 takes 57
// cycles for 32 of arithmetic).  Every wait and commit of the MMA thread is on that chain, which is why K and V
// pages share barriers and a page has one commit (65.5 -> 61.5 us at 2,048 tokens, 553 -> 510 us at 8,192).
// Variants that were built and measured slower at every length, and are not kept: two heads of a kv head per
// CTA with Q in tensor memory and K/V shared (one S buffer per head left the softmax warps idle during the
// head's own products: 748 against 588 us at 8,192 tokens); one CTA per SM with Q in tensor memory, two
// pages per step and four threads per row (83 against 63 us at 2,048 tokens, 887 against 1,113 TFLOP/s at
// 32,768); one CTA per SM with three score buffers of two pages (N 128), sixteen softmax warps, four threads per
// row, K and V units in two stages (75.8 against 61.5 us at 2,048 tokens, 635 against 518 at 8,192: its sixteen
// warps take their exponentials at the same time, 1,240 cycles for 32 per thread, which is the XU pipe's rate,
// and its MMAs still cost the issuing thread 90 to 115 cycles each beside them, as the N 64 ones do here, against
// 64 alone: two CTAs that drift apart overlap the two kinds of work better than one CTA in step with itself);
// the MMA warp running as a whole with only the MMAs predicated on one lane (no change); a start offset between
// an SM's two CTAs (no change); the scores issued by one thread and P V by another, K pages asked for by a softmax
// thread (68.5 us at 2,048, 590 at 8,192: the scores after next then wait for the P V product's commit to cross
// from one thread to the other, and each thread still takes ~95 cycles per MMA).  In isolation a thread needs
// ~59 cycles to issue one tcgen05.mma into an idle tensor core, whatever N (mma_probe.cu, patterns 4 and 5).
//
// Arithmetic as infer/forward.odin:88-115 (scale 1/sqrt(hd), causal bound t <= pos,
// maximum-subtracted softmax, weighted sum of values), in 32-bit except the bfloat16
// operands of the two products.  Every wait is bounded.
#include "attn_common.cuh"
#include <math_constants.h>

namespace {

using namespace attn;

constexpr int BQT = 128;  // query rows per CTA

struct PrefillTcParams {
    const bf16* q;
    size_t q_stride;
    bf16* out;
    size_t out_stride;
    int Hq, Hkv;
    const int* seq_start;
    const int* seq_len_after;
    const int* block_table;
    int bt_stride;
    int window;
    float scale_log2;
    int* error;
    int n_heads, n_seqs, n_tile_levels;  // the work: (head, sequence, tile) triples, heaviest tile level first
};

// The first wait that runs out records who it was: [which wait, head, sequence, tile, iteration,
// pages of the tile, thread].  Waits: 1 producer on a free K stage, 2 producer on a free V stage,
// 3 MMA on the first K pages, 4 MMA on P, 5 MMA on a landed slot (V and the K after next), 6 softmax on scores,
// 7 softmax on the previous P V (rescaling), 8 softmax on the last P V.
__device__ __noinline__ void report_attn(int* err, int what, int it, int n_pages) {
    if (err == nullptr) return;
    atomicOr(&err[7], 1 << what);           // every kind of wait that ran out
    atomicMax(&err[8 + what], it + 1);       // and the latest iteration it happened in
    if (atomicCAS(err, 0, what) == 0) {
        err[1] = (int)blockIdx.x; err[2] = (int)blockIdx.y; err[3] = (int)blockIdx.z; err[4] = it; err[5] = n_pages;
        err[6] = (int)threadIdx.x;
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// How far (in powers of two) a row's maximum may run ahead of the one its sums are scaled
// by before the accumulated O is rescaled.  Probabilities then reach at most 2^8, which
// bfloat16 and the 32-bit sums hold without loss; most pages need no rescaling at all.
constexpr float RESCALE_LAG = 8.0f;

#ifdef ODIN_TRACE
__device__ unsigned long long* odin_attn_clk = nullptr;
#endif

// The persistent CTAs' work counter and the count of CTAs that have left (see the kernel).
__device__ unsigned int g_prefill_next = 0, g_prefill_done = 0;

template <int HD>
__global__ void __launch_bounds__(320, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const PrefillTcParams p) {
    constexpr int NSUB = HD / 64;                 // 64-column sub-tiles of a row of head_dim
    constexpr int Q_SUB = BQT * 128;              // bytes of one [128 x 64] sub-tile of Q
    constexpr int KV_SUB = PAGE_T * 128;          // bytes of one [64 x 64] sub-tile of K or V
    constexpr int KV_TILE = NSUB * KV_SUB;
    constexpr int TMEM_COLS = (128 + HD) <= 256 ? 256 : 512;
    constexpr uint32_t S_COL = 0, O_COL = 128;    // S has two buffers of 64 columns

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + NSUB * Q_SUB;      // 2 stages
    uint8_t* sV = sK + 2 * KV_TILE;       // 2 stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * KV_TILE);
    // Every barrier completes once per use of ITS buffer or stage, and nobody can get two
    // completions ahead of its waiter: a parity wait cannot tell a phase from the one after next.
    uint64_t* kv_full = bars;          // [2] slot j (barrier j & 1): K page j and V page j - 2 landed (see the producer)
    uint64_t* s_full = bars + 2;       // [2] scores complete in S buffer b: the softmax may read, the K stage is free
    uint64_t* p_full = bars + 4;       // [2] P written over S buffer b, O rescaled if need be
    uint64_t* pv_done = bars + 6;      // [2] the P V product of one of the last two pages (buffer b) is complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_max = reinterpret_cast<float*>(bars + 16);  // [2 buffers][2 halves][128 rows]: the pair's exchange

    pdl_trigger();
    pdl_wait();
    if ((uint32_t)(smem - smem_raw) > 896u) {  // the shared-memory window is less aligned than assumed
        if (threadIdx.x == 0 && p.error != nullptr) atomicExch(p.error, 2);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 1) tc::tmem_alloc(tmem_slot, TMEM_COLS);
    if (threadIdx.x == 0) *abort_flag = 0;
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // The CTAs are persistent (two per SM) and take the (head, sequence, tile) triples themselves: the triples are
    // numbered with the tile level slowest and backwards (every sequence's latest, heaviest tiles first); a CTA
    // starts with the triple of its own number and then draws the next free number from a counter, so that unequal
    // sequences of a batch balance out.  Left to the hardware's block scheduler, a grid of one CTA per triple kept
    // an SM's second place empty until both of its first CTAs had ended (measured: the second wave of a 2,048-token
    // prompt began at 41 of 67 us, although CTAs had been ending since 26 us).  The counter lives in the library's
    // device image and is back at zero when the kernel ends (the last CTA out resets it), so the launches of a
    // process that use it must not overlap on the GPU: one stream, or events between streams.
    const long long total = (long long)p.n_heads * p.n_seqs * p.n_tile_levels;
    int* s_item = reinterpret_cast<int*>(tmem_slot + 2);
    bool first_item = true, first_ticket = true;
    for (;;) {
    if (threadIdx.x == 0)
        *s_item = first_ticket ? (int)blockIdx.x : (int)(gridDim.x + atomicAdd(&g_prefill_next, 1u));
    first_ticket = false;
    __syncthreads();
    const long long w = *s_item;
    __syncthreads();   // all have read the number before it is drawn again
    if (w >= total) break;
    odin_trace_mark(2);  // a triple begins (trace builds only)
    const int h = (int)(w % p.n_heads), seq = (int)((w / p.n_heads) % p.n_seqs);
    const int level = (int)(w / ((long long)p.n_heads * p.n_seqs));
    const int tok0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - tok0;
    const int n_tiles = (n_new + BQT - 1) / BQT;
    const int tile = p.n_tile_levels - 1 - level;
    if (tile >= n_tiles) continue;
    const int q0 = tile * BQT;
    const int rows = min(BQT, n_new - q0);
    const int len_after = p.seq_len_after[seq];
    const int pos0 = len_after - n_new + q0;
    const int kvh = h / (p.Hq / p.Hkv);
#ifdef ODIN_TRACE
    // Clock marks of the first triple's work (the heaviest tile of head 0), trace builds only: role 0 the MMA thread,
    // roles 1..8 the first lanes of the softmax warps; [role][n] = (clock << 8) | point.
    const bool traced = w == 0 && odin_attn_clk != nullptr;
    int clk_n = 0;
#define CLK(role, point)                                                                                         \
    do {                                                                                                         \
        if (traced && (role == 0 || lane == 0) && clk_n < 1024)                                                  \
            odin_attn_clk[((role) == 0 ? 0 : warp - 1) * 1024 + clk_n++] = ((unsigned long long)clock64() << 8) | (point); \
    } while (0)
#else
#define CLK(role, point) do {} while (0)
#endif

    int first_key = 0;
    if (p.window > 0 && pos0 - p.window + 1 > 0) first_key = pos0 - p.window + 1;
    const int page_a = first_key / PAGE_T, page_b = (pos0 + rows - 1) / PAGE_T;  // inclusive
    const int n_pages = page_b - page_a + 1;
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;

    if (threadIdx.x == 0) {
        // every triple starts with fresh barriers (all threads are past the last one's: the sync at the loop's end)
        if (!first_item)
            for (int i = 0; i < 8; ++i) tc::mbar_inval(&bars[i]);
        for (int i = 0; i < 8; ++i) tc::mbar_init(&bars[i], (i == 4 || i == 5) ? 8 : 1);   // p_full: one arrival per softmax warp
        tc::fence_barrier_init();
    }
    first_item = false;
    // Q: [128 x HD] in 64-column sub-tiles, each row's 16-byte chunks XOR-swizzled with the row
    for (int idx = threadIdx.x; idx < BQT * (HD / 8); idx += 320) {
        const int r = idx / (HD / 8), c = idx % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + (size_t)(tok0 + q0 + r) * p.q_stride + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(sQ + (c >> 3) * Q_SUB + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
    }
    tc::fence_proxy_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();

    if (warp == 0) {
        // ------------------------------------------------------------- producer
        if (lane == 0) {
            // Slot j brings K page j and V page j - 2 under one barrier: the MMA thread needs both at the same point
            // of its program (P V of page j - 2, then the scores of page j), and every wait costs it time that
            // nothing hides.  K page j goes where the scores of page j - 2 read, V page j - 2 where P V of page j - 4 read.
            // (Bringing the first two V pages with slots 0 and 1 gained nothing at 512 tokens and would let a barrier
            // run two phases ahead of the softmax threads that patch a short tile's last V page.)
            for (int j = 0; j < n_pages + 2; ++j) {
                const int b = j & 1;
                const bool has_k = j < n_pages, has_v = j >= 2;
                const int v_page = j - 2;
                // Slot j - 2 (the barrier's last use) must have landed AND the MMA thread must have seen it before the
                // barrier is armed again, or a parity wait would mistake the phase after next for its own.  The scores
                // of page j - 2 being complete says both (they were issued after that wait), and frees K's stage
                // and V's: P V of page j - 4 was issued before them, and a commit covers all MMAs before it.
                if (j >= 2 && !tc::mbar_wait(&s_full[b], ((j - 2) >> 1) & 1, abort_flag)) { report_attn(p.error, 1, j, n_pages); break; }
                tc::mbar_expect_tx(&kv_full[b], (has_k ? KV_TILE : 0) + (has_v ? KV_TILE : 0));
                if (has_v) {
                    const int row = (bt[page_a + v_page] * p.Hkv + kvh) * PAGE_T;
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub)
                        tc::tma_load_2d(sV + b * KV_TILE + sub * KV_SUB, &map_v, sub * 64, row, &kv_full[b]);
                }
                if (has_k) {
                    const int row = (bt[page_a + j] * p.Hkv + kvh) * PAGE_T;
#pragma unroll
                    for (int sub = 0; sub < NSUB; ++sub)
                        tc::tma_load_2d(sK + b * KV_TILE + sub * KV_SUB, &map_k, sub * 64, row, &kv_full[b]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = tc::make_idesc_bf16(BQT, PAGE_T);
            constexpr uint32_t idesc_o = tc::make_idesc_bf16_b_mn(BQT, HD);
            // The descriptors are made once per triple: a descriptor of a place `off` bytes further on is the
            // descriptor plus off / 16 (the address field holds bytes / 16 and cannot carry out of its 14 bits inside
            // the shared-memory window).  This thread shares its scheduler with softmax warps, so every instruction
            // between two MMAs costs it several cycles.
            const uint64_t q_desc = tc::make_smem_desc_sw128(tc::smem_u32(sQ));
            const uint64_t k_desc[2] = {tc::make_smem_desc_sw128(tc::smem_u32(sK)),
                                        tc::make_smem_desc_sw128(tc::smem_u32(sK + KV_TILE))};
            const uint64_t v_desc[2] = {tc::make_smem_desc_sw128_mn(tc::smem_u32(sV), KV_SUB, 1024),
                                        tc::make_smem_desc_sw128_mn(tc::smem_u32(sV + KV_TILE), KV_SUB, 1024)};
            // scores of page `it` into S buffer it & 1 (its K page landed with slot `it`, which the caller waited for)
            auto issue_s = [&](int it) {
                const int stage = it & 1;
                const uint64_t kd = stage ? k_desc[1] : k_desc[0];
                const uint32_t s_addr = tmem_base + S_COL + stage * PAGE_T;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    tc::umma_bf16(s_addr, q_desc + (uint64_t)(((k >> 2) * Q_SUB + (k & 3) * 32) >> 4),
                                  kd + (uint64_t)(((k >> 2) * KV_SUB + (k & 3) * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
                CLK(0, 16);  // S MMAs issued
                tc::umma_commit(&s_full[stage]);
                CLK(0, 10);  // S issued
            };
            bool ok = true;
            for (int j = 0; j < 2 && j < n_pages && ok; ++j) {
                if (!tc::mbar_wait(&kv_full[j], 0, abort_flag)) { report_attn(p.error, 3, j, n_pages); ok = false; break; }
                tc::fence_after_sync();
                issue_s(j);
            }
            for (int it = 0; it < n_pages && ok; ++it) {
                const int stage = it & 1;
                // the pages first: they land long before P is handed over, and what follows that hand-over is on the
                // chain that a page's time is made of
                if (!tc::mbar_wait(&kv_full[stage], ((it + 2) >> 1) & 1, abort_flag)) { report_attn(p.error, 5, it, n_pages); ok = false; break; }
                if (!tc::mbar_wait(&p_full[stage], (it >> 1) & 1, abort_flag)) { report_attn(p.error, 4, it, n_pages); ok = false; break; }
                tc::fence_after_sync();
                CLK(0, 11);  // P and V are there
                const uint64_t vd = stage ? v_desc[1] : v_desc[0];
                const uint32_t p_addr = tmem_base + S_COL + stage * PAGE_T;
                // P: 16 keys = 8 packed columns of the S buffer that the softmax overwrote.
                // V as stored: rows are keys (the MMA's K), head_dim contiguous (its N): MN-major.
                // 16 keys further = 16 rows of 128 bytes; 64-column sub-tiles KV_SUB apart; 8-key groups 1 KB apart.
                if (it > 0) {
#pragma unroll
                    for (int j = 0; j < PAGE_T / 16; ++j)
                        tc::umma_bf16_ts(tmem_base + O_COL, p_addr + j * 8, vd + (uint64_t)((j * 2048) >> 4), idesc_o, 1u);
                } else {
#pragma unroll
                    for (int j = 0; j < PAGE_T / 16; ++j)
                        tc::umma_bf16_ts(tmem_base + O_COL, p_addr + j * 8, vd + (uint64_t)((j * 2048) >> 4), idesc_o,
                                         j > 0 ? 1u : 0u);
                }
                CLK(0, 15);  // P V MMAs issued
                // One commit a page: the one behind the scores after next also tells that this P V is over;
                // only the last two pages, which no scores follow, have a commit of their own.
                if (it + 2 < n_pages) issue_s(it + 2);  // its S buffer was read before p_full(it)
                else tc::umma_commit(&pv_done[stage]);
                CLK(0, 13);  // P V and the scores after next issued
            }
        }
    } else {
        // ---------------------------- softmax: two threads per query row, 32 keys of a page each
        const int quarter = warp & 3;                 // the TMEM lanes this warp may touch
        const int half = (warp - 2) >> 2;             // warps 2..5: keys 0..31 of a page, warps 6..9: keys 32..63
        const int row = quarter * 32 + lane;
        const int pos = pos0 + row;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float scale = p.scale_log2;
        float m_run = -CUDART_INF_F;   // the maximum that the sums and O are scaled by (in log2 units)
        float l_run = 0.f;             // this thread's share of the row's sum
        bool ok = true;
        for (int it = 0; it < n_pages; ++it) {
            const int pg = page_a + it, stage = it & 1;
            if (!tc::mbar_wait(&s_full[stage], (it >> 1) & 1, abort_flag)) { report_attn(p.error, 6, it, n_pages); ok = false; break; }
            tc::fence_after_sync();
            CLK(1, 20);  // scores are there
            uint32_t sr[32];
            tc::tmem_ld32(tmem_base + lane_addr + S_COL + stage * PAGE_T + half * 32, sr);
            tc::tmem_ld_wait();
            CLK(1, 21);  // read
            const int key0 = pg * PAGE_T + half * 32;
            if ((pg * PAGE_T + PAGE_T - 1 > pos0) || p.window > 0) {  // a page on the diagonal or at the window's edge
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int t = key0 + c;
                    if (t > pos || (p.window > 0 && t <= pos - p.window)) sr[c] = 0xff800000u;  // -inf
                }
            }
            float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the row's maximum over both halves: exchange through shared memory within the warp pair
            s_max[(it & 1) * 256 + half * 128 + row] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            mx = fmaxf(mx, s_max[(it & 1) * 256 + (half ^ 1) * 128 + row]) * scale;
            CLK(1, 22);  // maximum known
            // move the scaling maximum only when the row's maximum ran ahead by more than the lag
            float corr = 1.0f;
            if (mx > m_run + RESCALE_LAG) {
                corr = ex2(m_run - mx);   // m_run = -inf gives 0
                m_run = mx;
            }
            const float neg_m = (m_run == -CUDART_INF_F) ? 0.f : -m_run;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float pv = ex2(fmaf(__uint_as_float(sr[c]), scale, neg_m));
                sr[c] = __float_as_uint(pv);
                sum4[c & 3] += pv;
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            CLK(1, 23);  // exponentials done
            // P: this thread's 32 keys as 16 packed words, written over the S buffer's columns
            {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) pk[c] = pack_bf16(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1]));
                tc::tmem_st16(tmem_base + lane_addr + S_COL + stage * PAGE_T + half * 16, pk);
            }
            if (it > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // O is touched only when the scaling maximum moved; the previous P V must be over first.
                // Each thread of the pair rescales half of the row's columns.
                // (told by the commit behind the scores of page it + 1, which were issued after it, or by its own)
                const bool pv_ok = (it + 1 < n_pages) ? tc::mbar_wait(&s_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag)
                                                      : tc::mbar_wait(&pv_done[(it - 1) & 1], 0, abort_flag);
                if (!pv_ok) { report_attn(p.error, 7, it, n_pages); ok = false; break; }
                tc::fence_after_sync();
#pragma unroll 1
                for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
                    uint32_t o[32];
                    tc::tmem_ld32(tmem_base + lane_addr + O_COL + c0, o);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
                    tc::tmem_st32(tmem_base + lane_addr + O_COL + c0, o);
                }
            }
            tc::tmem_st_wait();
            if (pg == page_b) {
                // Slots of the last page past the sequence's end may hold a stale Inf or NaN, and
                // 0 x NaN is NaN: clear those value rows (their probabilities are exactly 0).
                const int valid = len_after - pg * PAGE_T;
                if (valid < PAGE_T) {
                    tc::mbar_wait(&kv_full[stage], ((it + 2) >> 1) & 1, abort_flag);  // the tile (slot it + 2, the barrier's last) must have landed before it is patched
                    for (int idx = threadIdx.x - 64; idx < (PAGE_T - valid) * NSUB * 8; idx += 256) {
                        const int r = valid + idx / (NSUB * 8), rest = idx % (NSUB * 8);
                        *reinterpret_cast<uint4*>(sV + stage * KV_TILE + (rest >> 3) * KV_SUB + r * 128 + ((rest & 7) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    tc::fence_proxy_async();
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&p_full[stage]);
            CLK(1, 24);  // P handed over
        }
        if (ok && !tc::mbar_wait(&pv_done[(n_pages - 1) & 1], 0, abort_flag)) { report_attn(p.error, 8, n_pages, n_pages); ok = false; }
        if (ok) {
            tc::fence_after_sync();
            // the row's sum is the pair's two shares
            s_max[half * 128 + row] = l_run;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
            const float l_all = l_run + s_max[(half ^ 1) * 128 + row];
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            bf16* dst = p.out + (size_t)(tok0 + q0 + row) * p.out_stride + (size_t)h * HD;
#pragma unroll 1
            for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
                uint32_t o[32];
                tc::tmem_ld32(tmem_base + lane_addr + O_COL + c0, o);
                tc::tmem_ld_wait();
                if (row < rows) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 u;
                        u.x = pack_bf16(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
                        u.y = pack_bf16(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
                        u.z = pack_bf16(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
                        u.w = pack_bf16(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * c) = u;
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();   // the triple is done: its barriers, Q and stages are free
    if (*abort_flag) break;
    }  // the next triple

    odin_trace_mark(9);  // the CTA's work is done (trace builds only)
    if (threadIdx.x == 0) {
        if (*abort_flag && p.error != nullptr) atomicCAS(p.error, 0, 99);
        if (atomicAdd(&g_prefill_done, 1u) == gridDim.x - 1) {  // the last CTA out: the counters start from zero again
            g_prefill_next = 0;
            g_prefill_done = 0;
            __threadfence();
        }
    }
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int* tc_error_flag() {
    static int* flag = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&flag, 32 * sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, 32 * sizeof(int));
        else flag = nullptr;
    });
    return flag;
}

template <int HD>
int launch_prefill_tc(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillTcParams& p, int n_seqs, int max_new,
                      cudaStream_t s) {
    // tiles + barriers + slack for the 1 KB alignment; two CTAs of head size 128 just fit an SM's 228 KB
    constexpr int SMEM = (HD / 64) * BQT * 128 + 4 * PAGE_T * HD * 2 + 128 + 2048 + 896;  // (barriers 128, exchange 2048, alignment 896)
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    PrefillTcParams q = p;
    q.n_heads = p.Hq; q.n_seqs = n_seqs; q.n_tile_levels = (max_new + BQT - 1) / BQT;
    const long long total = (long long)q.n_heads * q.n_seqs * q.n_tile_levels;
    if (total > (1LL << 30)) return ODIN_ERR_UNSUPPORTED;  // the work counter is 32 bits wide
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int grid = (int)(total < 2LL * sms ? total : 2LL * sms);
    odin_launch(attn_prefill_tc_kernel<HD>, dim3(grid), dim3(320), (size_t)SMEM, s, mk, mv, q);
    ODIN_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// Same arguments as odin_attention_prefill; the output rows must be 16-byte aligned.
extern "C" int odin_attention_prefill_tc(const void* q, long long q_row_stride, void* out, long long out_row_stride,
                                         int n_seqs, int max_new, int Hq, int Hkv, int hd, const void* k_cache,
                                         const void* v_cache, int n_pages, const int* seq_start,
                                         const int* seq_len_after, const int* block_table, int bt_stride, int window,
                                         void* stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0) return ODIN_ERR_BAD_ARG;
    if ((q_row_stride % 8) || (((uintptr_t)q) & 15) || (out_row_stride % 8) || (((uintptr_t)out) & 15))
        return ODIN_ERR_UNSUPPORTED;
    CUtensorMap mk, mv;
    int rc;
    const long long rows = (long long)n_pages * Hkv * PAGE_T;
    if ((rc = cache_map(&mk, k_cache, rows, hd))) return rc;
    if ((rc = cache_map(&mv, v_cache, rows, hd))) return rc;
    PrefillTcParams p;
    p.q = (const bf16*)q; p.q_stride = (size_t)q_row_stride;
    p.out = (bf16*)out; p.out_stride = (size_t)out_row_stride;
    p.Hq = Hq; p.Hkv = Hkv;
    p.seq_start = seq_start; p.seq_len_after = seq_len_after;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.window = window;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    p.error = tc_error_flag();
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch_prefill_tc<64>(mk, mv, p, n_seqs, max_new, s);
    if (hd == 128) return launch_prefill_tc<128>(mk, mv, p, n_seqs, max_new, s);
    return ODIN_ERR_UNSUPPORTED;
}

#ifdef ODIN_TRACE
extern "C" int odin_attention_prefill_tc_set_clk(void* buf) {
    return cudaMemcpyToSymbol(odin_attn_clk, &buf, sizeof(buf)) != cudaSuccess;
}
#endif

extern "C" int odin_attention_prefill_tc_error_detail(int* out8) {
    int* f = tc_error_flag();
    if (f == nullptr) return 0;
    if (cudaMemcpy(out8, f, 32 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return out8[0];
}

extern "C" int odin_attention_prefill_tc_error() {
    int* f = tc_error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) {
        cudaMemset(f, 0, 32 * sizeof(int));
        // a launch that gave up may have left the work counters anywhere
        const unsigned int zero = 0;
        cudaMemcpyToSymbol(g_prefill_next, &zero, sizeof(zero));
        cudaMemcpyToSymbol(g_prefill_done, &zero, sizeof(zero));
    }
    return v;
}

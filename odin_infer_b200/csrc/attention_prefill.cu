// Causal grouped-query attention of whole prompts (or pieces of them) over the paged
// bfloat16 cache: a flash-attention kernel with the keys and values of one cache
// page (64 tokens) per iteration.
//
// One CTA of 4 warps takes 64 consecutive query tokens of one sequence and one query
// head; each warp owns 16 query rows.  K and V pages arrive in shared memory by TMA
// (2-D tiles of the cache seen as [rows, head_dim], 128-byte swizzle, two stages), Q
// is read once with plain loads into the same swizzle.  S = Q K^T and O += P V run on
// the tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit accumulate); the running
// maximum, the sums and the rescaling of the softmax are kept in 32-bit registers.
// The keys of this step's own tokens are already in the cache (written by the head
// preparation kernel), so a prompt that continues from a non-zero position is
// handled like one that starts at 0.
//
// Arithmetic follows infer/forward.odin:88-115 (scale 1/sqrt(hd), causal bound t <= pos,
// softmax with the maximum subtracted, weighted sum of values); scale and log2(e) are
// folded so that the exponentials are exp2.  A window > 0 hides keys t <= pos - window.
#include "attn_common.cuh"
#include <math_constants.h>

namespace {

using namespace attn;

constexpr int BQ = 64;      // query rows per CTA
constexpr int NWARP = 4;

struct PrefillParams {
    const bf16* q;
    size_t q_stride;
    bf16* out;
    size_t out_stride;
    int Hq, Hkv;
    const int* seq_start;      // [n_seqs + 1] first token row of each sequence
    const int* seq_len_after;  // [n_seqs] length of each sequence once the step is done
    const int* block_table;
    int bt_stride;
    int window;
    float scale_log2;
    int* error;
};

template <int HD>
__global__ void __launch_bounds__(NWARP * 32)
attn_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const PrefillParams p) {
    constexpr int TILE = PAGE_T * HD * 2;  // bytes of one K (or V) page of one head
    constexpr int KB = HD / 16;            // k-blocks of Q K^T
    constexpr int NB_S = PAGE_T / 8;       // 8-key blocks of S
    constexpr int NB_O = HD / 8;           // 8-dim blocks of O
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = smem + TILE;           // 2 stages
    uint8_t* sV = smem + 3 * TILE;       // 2 stages
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + 5 * TILE);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(full + 2);

    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y, h = blockIdx.z;
    const int tok0 = p.seq_start[seq], n_new = p.seq_start[seq + 1] - tok0;
    const int n_tiles = (n_new + BQ - 1) / BQ;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // the heaviest (latest) tiles first
    if (tile >= n_tiles) return;
    const int q0 = tile * BQ;                        // first query row of the tile within this step's tokens
    const int rows = min(BQ, n_new - q0);
    const int len_after = p.seq_len_after[seq];
    const int pos0 = len_after - n_new + q0;  // position of the tile's first query
    const int kvh = h / (p.Hq / p.Hkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int first_key = 0;
    if (p.window > 0 && pos0 - p.window + 1 > 0) first_key = pos0 - p.window + 1;
    const int page_a = first_key / PAGE_T, page_b = (pos0 + rows - 1) / PAGE_T;  // inclusive
    const int* bt = p.block_table + (size_t)seq * p.bt_stride;

    if (threadIdx.x == 0) {
        tc::mbar_init(&full[0], 1);
        tc::mbar_init(&full[1], 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    // Q tile: plain loads into the swizzled layout (rows past the end are zero)
    for (int idx = threadIdx.x; idx < BQ * (HD / 8); idx += NWARP * 32) {
        const int r = idx / (HD / 8), c = idx % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(p.q + (size_t)(tok0 + q0 + r) * p.q_stride + (size_t)h * HD + c * 8);
        *reinterpret_cast<uint4*>(sQ + tile_off(r, c * 8)) = v;
    }
    __syncthreads();

    auto issue = [&](int page_idx, int stage) {
        const int page = bt[page_idx];
        const int row = (page * p.Hkv + kvh) * PAGE_T;  // row of the cache seen as [pages*Hkv*64, HD]
        tc::mbar_expect_tx(&full[stage], 2 * TILE);
#pragma unroll
        for (int sub = 0; sub < HD / 64; ++sub) {
            tc::tma_load_2d(sK + stage * TILE + sub * 8192, &map_k, sub * 64, row, &full[stage]);
            tc::tma_load_2d(sV + stage * TILE + sub * 8192, &map_v, sub * 64, row, &full[stage]);
        }
    };
    if (threadIdx.x == 0) {
        issue(page_a, 0);
        if (page_a + 1 <= page_b) issue(page_a + 1, 1);
    }

    float o[NB_O][4];
#pragma unroll
    for (int i = 0; i < NB_O; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    const int row_a = warp * 16 + (lane >> 2);  // this thread's rows within the tile: row_a and row_a + 8
    const int pos_a = pos0 + row_a, pos_b = pos_a + 8;
    const uint32_t sQ_u = tc::smem_u32(sQ);

    bool ok = true;
    for (int pg = page_a; pg <= page_b; ++pg) {
        const int stage = (pg - page_a) & 1;
        const uint32_t phase = ((pg - page_a) >> 1) & 1;
        if (!tc::mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
        const uint32_t sK_u = tc::smem_u32(sK + stage * TILE), sV_u = tc::smem_u32(sV + stage * TILE);
        if (pg == page_b) {
            // Slots of the last page beyond the sequence's end hold whatever an earlier owner
            // left there.  Their probabilities are exactly 0, but 0 times a stale Inf or NaN
            // is NaN, so those value rows are cleared (the scores are overwritten by the mask).
            const int valid = len_after - pg * PAGE_T;
            if (valid < PAGE_T) {
                for (int idx = threadIdx.x; idx < (PAGE_T - valid) * (HD / 8); idx += NWARP * 32) {
                    const int r = valid + idx / (HD / 8), c = idx % (HD / 8);
                    *reinterpret_cast<uint4*>(sV + stage * TILE + tile_off(r, c * 8)) = make_uint4(0, 0, 0, 0);
                }
                __syncthreads();
            }
        }

        // ---- S = Q K^T for this warp's 16 rows and the page's 64 keys
        float s[NB_S][4];
#pragma unroll
        for (int i = 0; i < NB_S; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            uint32_t a[4];
            ldmatrix_x4(a, sQ_u + tile_off(warp * 16 + (lane & 15), kb * 16 + (lane >> 4) * 8));
#pragma unroll
            for (int nb2 = 0; nb2 < NB_S / 2; ++nb2) {
                uint32_t b[4];
                // matrices: (keys +0..7, k 0..7), (keys +0..7, k 8..15), (keys +8..15, k 0..7), (keys +8..15, k 8..15)
                ldmatrix_x4(b, sK_u + tile_off(nb2 * 16 + (lane & 7) + ((lane >> 4) << 3), kb * 16 + ((lane >> 3) & 1) * 8));
                mma_bf16(s[2 * nb2], a, b[0], b[1]);
                mma_bf16(s[2 * nb2 + 1], a, b[2], b[3]);
            }
        }
        // ---- scale, mask, online softmax
        const int key0 = pg * PAGE_T + (lane & 3) * 2;
        const bool need_mask = (pg * PAGE_T + PAGE_T - 1 > pos0 + warp * 16) || p.window > 0;
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nb = 0; nb < NB_S; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v = s[nb][j] * p.scale_log2;
                if (need_mask) {
                    const int t = key0 + nb * 8 + (j & 1);
                    const int pos = (j < 2) ? pos_a : pos_b;
                    if (t > pos || (p.window > 0 && t <= pos - p.window)) v = -CUDART_INF_F;
                }
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
            m_use[r] = (m_new == -CUDART_INF_F) ? 0.f : m_new;  // a row that has seen no key yet
            corr[r] = exp2f(m_run[r] - m_use[r]);               // m_run = -inf gives 0
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nb = 0; nb < NB_S; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float pv = exp2f(s[nb][j] - m_use[j >> 1]);
                s[nb][j] = pv;
                l_run[j >> 1] += pv;
            }
        }
#pragma unroll
        for (int i = 0; i < NB_O; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // ---- O += P V
#pragma unroll
        for (int kb = 0; kb < PAGE_T / 16; ++kb) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
            a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
            a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
            a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
            for (int nb2 = 0; nb2 < NB_O / 2; ++nb2) {
                uint32_t b[4];
                // transposed loads: (keys +0..7, dims +0..7), (keys +8..15, dims +0..7), (keys +0..7, dims +8..15), (keys +8..15, dims +8..15)
                ldmatrix_x4_trans(b, sV_u + tile_off(kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), nb2 * 16 + (lane >> 4) * 8));
                mma_bf16(o[2 * nb2], a, b[0], b[1]);
                mma_bf16(o[2 * nb2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // everyone is done with this stage
        if (threadIdx.x == 0 && pg + 2 <= page_b) issue(pg + 2, stage);
    }

    if (threadIdx.x == 0 && (!ok || *abort_flag) && p.error != nullptr) atomicExch(p.error, 1);
    if (!ok) return;
    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_a = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f;
    const float inv_b = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    const int col = (lane & 3) * 2;
    if (row_a < rows) {
        bf16* dst = p.out + (size_t)(tok0 + q0 + row_a) * p.out_stride + (size_t)h * HD + col;
#pragma unroll
        for (int i = 0; i < NB_O; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
    }
    if (row_a + 8 < rows) {
        bf16* dst = p.out + (size_t)(tok0 + q0 + row_a + 8) * p.out_stride + (size_t)h * HD + col;
#pragma unroll
        for (int i = 0; i < NB_O; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

// ------------------------------------------------------------------ host side
int* error_flag() {
    static int* flag = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&flag, sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, sizeof(int));
        else flag = nullptr;
    });
    return flag;
}

template <int HD>
int launch_prefill(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, int n_seqs, int max_new,
                   cudaStream_t s) {
    constexpr int SMEM = 5 * PAGE_T * HD * 2 + 1024 + 64;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((max_new + BQ - 1) / BQ, n_seqs, p.Hq);
    odin_launch(attn_prefill_kernel<HD>, grid, dim3(NWARP * 32), (size_t)SMEM, s, mk, mv, p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

}  // namespace

extern "C" int odin_attention_prefill_supported(int hd) { return hd == 64 || hd == 128; }

// q: this step's query rows [T, Hq*hd] (row stride q_row_stride), sequence b owning rows
// [seq_start[b], seq_start[b+1]); its last row sits at position seq_len_after[b] - 1.
// max_new: the largest number of rows any sequence brings (sizes the grid).
// k_cache, v_cache: one layer's [pages][Hkv][64][hd] bfloat16; n_pages of them.
extern "C" int odin_attention_prefill(const void* q, long long q_row_stride, void* out, long long out_row_stride,
                                      int n_seqs, int max_new, int Hq, int Hkv, int hd, const void* k_cache,
                                      const void* v_cache, int n_pages, const int* seq_start,
                                      const int* seq_len_after, const int* block_table, int bt_stride, int window,
                                      void* stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (Hkv <= 0 || Hq % Hkv != 0) return ODIN_ERR_BAD_ARG;
    if (n_seqs > 65535 || Hq > 65535) return ODIN_ERR_UNSUPPORTED;
    if ((q_row_stride % 8) || (((uintptr_t)q) & 15) || (out_row_stride % 2)) return ODIN_ERR_UNSUPPORTED;
    CUtensorMap mk, mv;
    int rc;
    const long long rows = (long long)n_pages * Hkv * PAGE_T;
    if ((rc = cache_map(&mk, k_cache, rows, hd))) return rc;
    if ((rc = cache_map(&mv, v_cache, rows, hd))) return rc;
    PrefillParams p;
    p.q = (const bf16*)q; p.q_stride = (size_t)q_row_stride;
    p.out = (bf16*)out; p.out_stride = (size_t)out_row_stride;
    p.Hq = Hq; p.Hkv = Hkv;
    p.seq_start = seq_start; p.seq_len_after = seq_len_after;
    p.block_table = block_table; p.bt_stride = bt_stride;
    p.window = window;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    p.error = error_flag();
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64) return launch_prefill<64>(mk, mv, p, n_seqs, max_new, s);
    if (hd == 128) return launch_prefill<128>(mk, mv, p, n_seqs, max_new, s);
    return ODIN_ERR_UNSUPPORTED;
}

extern "C" int odin_attention_prefill_error() {
    int* f = error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(f, 0, sizeof(int));
    return v;
}

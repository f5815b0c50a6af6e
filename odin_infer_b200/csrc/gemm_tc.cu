// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to shared
// memory by TMA in the 128-byte swizzle, a ring of stages, and a persistent CTA per
// SM that walks over output tiles with two accumulators, so the epilogue of one
// tile overlaps the products of the next.
//
// Roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and
// issues the MMAs (one lane), warps 2..5 read the accumulator back and store.
// This is the kernel of steps of up to 128 tokens (mode 1); products of more tokens run on
// pairs of SMs (gemm_tc2.cu).
//
// The product is computed as D = X * Y^T with X on the 128-row side of the MMA and
// Y on its N side.  Two modes map the matrices to X and Y:
//   mode 0 (many tokens):  X = A (tokens),  Y = W;  D[i][j] -> C[i][j]
//   mode 1 (few tokens):   X = W,           Y = A;  D[i][j] -> C[j][i]
// Mode 1 puts the weight rows on the wide side, so decoding a handful of tokens
// still fills the MMA and streams each weight exactly once.
//
// Split-K: the K range can be cut into `n_split` parts, each written as a 32-bit
// partial sum to its own slice of the output ([n_split][M][N]); the consumer adds
// them in a fixed order.  Which part a CTA takes never depends on M, so a token's
// result does not depend on what else is in the batch.
//
// Weights staged in tensor memory (mode 1, `staged` > 0).  A product of few tokens starts while the
// kernel before it still runs and can fetch weights, but nothing else, until that kernel is done; its
// ring of stages is full after ~3 us of the 3 to 9 us that it waits.  So the first `staged` K blocks of
// the CTA's first item pass through the ring into tensor memory (tcgen05.cp, 32 columns a block beside
// the accumulators), the ring fills again behind them, and when the wait ends up to 400 KB of the CTA's
// weights are on the SM.  Their MMAs read A from tensor memory and the tokens' tiles, fetched after the
// wait, from a small area of their own.  The K blocks are multiplied in the same order either way.
//
// In the reference this is the weight-times-activation product of every layer
// (infer/matmul.odin:77-109, one row-dot per thread on the CPU; gemv kernels in
// infer/metal.odin:76-109 on the GPU).
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "tc_common.cuh"

namespace {

constexpr int BM = 128;  // rows of X per tile (MMA M)
constexpr int BK = 64;   // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int ACC_BUFS = 2;

struct GemmParams {
    void* out;             // C (or the partial-sum slices)
    long long ldc;         // leading dimension of C in elements
    long long split_stride;  // elements between partial-sum slices
    int rows_x, rows_y;    // rows of X and Y
    int K;
    int tiles_x, tiles_y;
    int n_split, kb_per_split, kb_total;
    int dual_offset;       // DUAL: first row of the second Y tile's matrix half
    int stages;            // length of the ring of stages (0: as many as fit)
    int staged;            // mode 1: K blocks of a CTA's first item whose weights wait in tensor memory (see the kernel)
    int* error;            // set when a wait runs out
};

// DUAL: two Y tiles per stage (rows [j, j+BN) and [dual_offset + j, dual_offset + j + BN) of Y) and
// two accumulators side by side, for the gate and up halves of a fused SwiGLU matrix.
template <int BN, bool DUAL = false>
struct Cfg {
    static constexpr int NY = DUAL ? 2 : 1;
    static constexpr int ACC_W = NY * BN;  // accumulator columns per buffer
    static constexpr int STAGE_X = BM * BK * 2;
    static constexpr int STAGE_Y1 = BN * BK * 2;
    static constexpr int STAGE_Y = NY * STAGE_Y1;
    static constexpr int STAGE = STAGE_X + STAGE_Y;
    static constexpr int STAGES = (196608 / STAGE) > 10 ? 10 : (196608 / STAGE);
    static constexpr int TMEM_COLS = (ACC_BUFS * ACC_W) < 32 ? 32 : (ACC_BUFS * ACC_W);
    static constexpr int SMEM = STAGES * STAGE + 1024 /*alignment*/ + 256 /*barriers*/;
};

// The first wait that runs out records who it was: [which wait, block, work item, K block, stage or
// accumulator, mode, tile width, grid size].  Waits: 1 producer on a free stage, 2 MMA on a free
// accumulator, 3 MMA on a landed stage, 4 epilogue on a complete accumulator.
__device__ __noinline__ void report(int* err, int what, int item, int kb, int slot, int mode, int bn) {
    if (err == nullptr) return;
    if (atomicCAS(err, 0, what) == 0) {
        err[1] = (int)blockIdx.x; err[2] = item; err[3] = kb; err[4] = slot; err[5] = mode; err[6] = bn;
        err[7] = (int)gridDim.x;
    }
}

template <typename TO>
__device__ __forceinline__ void store_vec(TO* dst, const uint32_t* r, int n);

// n floats (bit patterns in r) to consecutive elements, vectorised when aligned
template <>
__device__ __forceinline__ void store_vec<float>(float* dst, const uint32_t* r, int n) {
    if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
        for (int i = 0; i < n; ++i) dst[i] = __uint_as_float(r[i]);
    }
}

template <>
__device__ __forceinline__ void store_vec<bf16>(bf16* dst, const uint32_t* r, int n) {
    if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]),
                                                         __uint_as_float(r[8 * i + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[0], p[1], p[2], p[3]);
        }
    } else {
        for (int i = 0; i < n; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

template <int BN, int MODE, typename TO, bool DUAL = false>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
               const __grid_constant__ CUtensorMap map_y3, const GemmParams p) {
    using C = Cfg<BN, DUAL>;
    static_assert(!DUAL || MODE == 0, "the SwiGLU epilogue exists for mode 0 only");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t n_stages = (uint32_t)p.stages;  // at most C::STAGES: the ring may be shorter to leave shared memory to a neighbour
    const int n_staged = (MODE == 1) ? p.staged : 0;
    uint8_t* y_staged = smem + n_stages * C::STAGE;  // [staged] token tiles of the K blocks whose weights wait in tensor memory
    uint64_t* bars = reinterpret_cast<uint64_t*>(y_staged + n_staged * C::STAGE_Y1);
    uint64_t* full = bars;                        // [STAGES] TMA landed
    uint64_t* empty = bars + C::STAGES;           // [STAGES] MMAs that read the stage are done
    uint64_t* acc_full = bars + 2 * C::STAGES;    // [ACC_BUFS] accumulator complete
    uint64_t* acc_empty = acc_full + ACC_BUFS;    // [ACC_BUFS] accumulator read back
    uint64_t* y_full = acc_empty + ACC_BUFS;      // the token tiles of the staged K blocks have landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(y_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_trigger();  // the next kernel may take its place; it waits for this one before it touches memory

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {  // all of them: the places are there whatever the ring's length
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < ACC_BUFS; ++a) {
            tc::mbar_init(&acc_full[a], 1);
            tc::mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
        }
        tc::mbar_init(y_full, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_x);
        tc::prefetch_tensormap(&map_y);
        if (MODE == 1 && p.staged > 0) tc::prefetch_tensormap(&map_y3);
    }
    // with staged weights the CTA takes all of tensor memory: 32 columns a staged block beside the accumulators
    const uint32_t tmem_cols = n_staged > 0 ? 512u : (uint32_t)C::TMEM_COLS;
    if (warp == 1) tc::tmem_alloc(tmem_slot, tmem_cols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_staged = tmem_base + ACC_BUFS * C::ACC_W;

    const long long n_items = (long long)p.tiles_x * p.tiles_y * p.n_split;
    // the CTA's first item: how many of its K blocks are staged (t_first), how many more the ring takes before the wait
    int first_kb0 = 0, t_first = 0, r_first = 0, first_tx = 0, first_ty = 0;
    if (MODE == 1 && (long long)blockIdx.x < n_items) {
        const long long w = blockIdx.x;
        const int s0 = (int)(w % p.n_split);
        first_tx = (int)((w / p.n_split) % p.tiles_x);
        first_ty = (int)((w / p.n_split) / p.tiles_x);
        first_kb0 = s0 * p.kb_per_split;
        const int nk = min(p.kb_total, first_kb0 + p.kb_per_split) - first_kb0;
        t_first = min(n_staged, nk);
        r_first = min((int)n_stages, nk - t_first);
    }

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // Weights are constant: in mode 1 (X = weights) the first stages of the first tile
            // are requested before the wait for the previous kernel, whose output is only Y.
            int pre = 0;  // K blocks of the first item requested before the wait
            if (MODE == 1 && (long long)blockIdx.x < n_items) {
                // the staged blocks' weights: through the ring, which the MMA warp empties into tensor memory
                for (int j = 0; j < t_first && ok; ++j) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report(p.error, 1, (int)blockIdx.x, first_kb0 + j, stage, MODE, BN); ok = false; break; }
                    tc::mbar_expect_tx(&full[stage], C::STAGE_X);
                    tc::tma_load_2d(smem + stage * C::STAGE, &map_x, (first_kb0 + j) * BK, first_tx * BM, &full[stage]);
                    if (++stage == n_stages) { stage = 0; phase ^= 1; }
                }
                // then the ring's own blocks: their weights now, their tokens after the wait
                const uint32_t stage_r = stage, phase_r = phase;
                for (int i = 0; i < r_first && ok; ++i) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report(p.error, 1, (int)blockIdx.x, first_kb0 + t_first + i, stage, MODE, BN); ok = false; break; }
                    tc::mbar_expect_tx(&full[stage], C::STAGE);
                    tc::tma_load_2d(smem + stage * C::STAGE, &map_x, (first_kb0 + t_first + i) * BK, first_tx * BM, &full[stage]);
                    if (++stage == n_stages) { stage = 0; phase ^= 1; }
                }
                pdl_wait();
                if (ok) {
                    if (t_first > 0) {
                        // the staged blocks' token tiles in one copy: a box of `staged` K blocks (those beyond the
                        // item's are read and not used)
                        tc::mbar_expect_tx(y_full, (uint32_t)n_staged * C::STAGE_Y1);
                        tc::tma_load_3d(y_staged, &map_y3, 0, first_ty * BN, first_kb0, y_full);
                    }
                    uint32_t st = stage_r;
                    for (int i = 0; i < r_first; ++i) {
                        tc::tma_load_2d(smem + st * C::STAGE + C::STAGE_X, &map_y, (first_kb0 + t_first + i) * BK, first_ty * BN, &full[st]);
                        if (++st == n_stages) st = 0;
                    }
                }
                (void)phase_r;
                pre = t_first + r_first;
            } else {
                pdl_wait();
            }
            for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
                const int s = (int)(w % p.n_split);
                const long long rest = w / p.n_split;
                const int tx = (int)(rest % p.tiles_x), ty = (int)(rest / p.tiles_x);
                const int kb0 = s * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                for (int kb = kb0 + pre; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report(p.error, 1, (int)w, kb, stage, MODE, BN); ok = false; break; }
                    uint8_t* sx = smem + stage * C::STAGE;
                    uint8_t* sy = sx + C::STAGE_X;
                    tc::mbar_expect_tx(&full[stage], C::STAGE);
                    tc::tma_load_2d(sx, &map_x, kb * BK, tx * BM, &full[stage]);
                    tc::tma_load_2d(sy, &map_y, kb * BK, ty * BN, &full[stage]);
                    if (DUAL) tc::tma_load_2d(sy + C::STAGE_Y1, &map_y, kb * BK, p.dual_offset + ty * BN, &full[stage]);
                    if (++stage == n_stages) { stage = 0; phase ^= 1; }
                }
                pre = 0;
            }
            odin_trace_mark(6, true);  // every load of this CTA is requested
            if (!ok) {
                // aborted: let the copies already in flight land before the CTA's memory is released
                for (uint32_t s2 = 0; s2 < n_stages; ++s2)
                    for (uint32_t i = 0; i < 4096; ++i)
                        if (tc::mbar_try_wait(&full[s2], 0) || tc::mbar_try_wait(&full[s2], 1)) break;
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer
        if (MODE == 1) {
            // The whole warp walks the loop and one elected lane issues: in code that a single lane
            // runs alone the per-stage cost (wait, descriptors, four MMAs, commit) was 520 cycles
            // against 350 this way, which matters when an MMA is as short as with 16 tokens.  The
            // next stage's barrier is tested before this stage's MMAs go out, so that its latency
            // hides behind them.
            constexpr uint32_t idesc = tc::make_idesc_bf16(BM, BN);
            uint32_t stage = 0, phase = 0;
            uint32_t local = 0;
            bool ok = true;
            // the staged blocks' weights: from the ring into tensor memory as they land, before the wait ends
            for (int j = 0; j < t_first && ok; ++j) {
                ok = __all_sync(0xffffffffu, tc::mbar_wait(&full[stage], phase, abort_flag));
                if (!ok) { if (lane == 0) report(p.error, 3, (int)blockIdx.x, first_kb0 + j, stage, MODE, BN); break; }
                tc::fence_after_sync();
                if (tc::elect_one()) {
                    const uint64_t dx = tc::make_smem_desc_sw128(tc::smem_u32(smem + stage * C::STAGE));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) tc::tmem_cp_128x256b(tmem_staged + 32 * j + 8 * k, dx + 2 * k);
                    tc::umma_commit(&empty[stage]);
                }
                __syncwarp();
                if (++stage == n_stages) { stage = 0; phase ^= 1; }
            }
            pdl_wait();  // nothing can be multiplied before the previous kernel's output exists: sleep, do not spin
            bool ready = false;
            for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++local) {
                const int s = (int)(w % p.n_split);
                const int kb0 = s * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
                ok = __all_sync(0xffffffffu, tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag));
                if (!ok) { if (lane == 0) report(p.error, 2, (int)w, -1, (int)acc, MODE, BN); break; }
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * C::ACC_W;
                int staged_here = 0;
                if (local == 0 && t_first > 0) {
                    // the staged blocks: A from tensor memory, the tokens' tiles from their own area
                    ok = __all_sync(0xffffffffu, tc::mbar_wait(y_full, 0, abort_flag));
                    if (!ok) { if (lane == 0) report(p.error, 3, (int)w, kb0, -1, MODE, BN); break; }
                    tc::fence_after_sync();
                    if (tc::elect_one()) {
                        for (int j = 0; j < t_first; ++j) {
                            const uint64_t dy = tc::make_smem_desc_sw128(tc::smem_u32(y_staged + j * C::STAGE_Y1));
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                tc::umma_bf16_ts(tmem_d, tmem_staged + 32 * j + 8 * k, dy + 2 * k, idesc, (j > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    __syncwarp();
                    staged_here = t_first;
                }
                for (int kb = kb0 + staged_here; kb < kb1; ++kb) {
                    if (!ready) ready = tc::mbar_wait(&full[stage], phase, abort_flag);
                    ok = __all_sync(0xffffffffu, ready);
                    if (!ok) { if (lane == 0) report(p.error, 3, (int)w, kb, stage, MODE, BN); break; }
                    tc::fence_after_sync();
                    const uint32_t cur = stage;
                    if (++stage == n_stages) { stage = 0; phase ^= 1; }
                    ready = __all_sync(0xffffffffu, tc::mbar_test_wait(&full[stage], phase));
                    if (tc::elect_one()) {
                        const uint32_t ax = tc::smem_u32(smem + cur * C::STAGE);
                        const uint64_t dx = tc::make_smem_desc_sw128(ax);
                        const uint64_t dy = tc::make_smem_desc_sw128(ax + C::STAGE_X);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // +32 bytes per K step inside the 128-byte swizzle row: +2 in 16-byte units
                            tc::umma_bf16(tmem_d, dx + 2 * k, dy + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        }
                        if (DUAL) {
                            const uint64_t dy2 = tc::make_smem_desc_sw128(ax + C::STAGE_X + C::STAGE_Y1);
#pragma unroll
                            for (int k = 0; k < BK / UMMA_K; ++k)
                                tc::umma_bf16(tmem_d + BN, dx + 2 * k, dy2 + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        }
                        tc::umma_commit(&empty[cur]);
                    }
                    __syncwarp();
                }
                if (ok && tc::elect_one()) tc::umma_commit(&acc_full[acc]);
                __syncwarp();
                if (local == 0 && lane == 0) odin_trace_mark(2, true);  // the first item's MMAs are issued
            }
            if (lane == 0) odin_trace_mark(3, true);  // the last commit is issued
        } else {
            // many tokens: an MMA of 256 columns takes 128 cycles, the issuing lane is never the limit,
            // and a single lane that walks the loop alone measured 2 % faster than the converged warp
            if (lane == 0) {
                // DUAL: the gate tile and the up tile lie one after the other in shared memory: one MMA over
                // both, gate in the accumulator's columns [0, BN), up in [BN, 2 BN)
                constexpr uint32_t idesc = tc::make_idesc_bf16(BM, DUAL ? 2 * BN : BN);
                uint32_t stage = 0, phase = 0;
                uint32_t local = 0;
                bool ok = true;
                pdl_wait();  // nothing can be multiplied before the previous kernel's output exists: sleep, do not spin
                for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++local) {
                    const int s = (int)(w % p.n_split);
                    const int kb0 = s * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                    const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
                    if (!tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { report(p.error, 2, (int)w, -1, (int)acc, MODE, BN); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t tmem_d = tmem_base + acc * C::ACC_W;
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!tc::mbar_wait(&full[stage], phase, abort_flag)) { report(p.error, 3, (int)w, kb, stage, MODE, BN); ok = false; break; }
                        tc::fence_after_sync();
                        const uint32_t ax = tc::smem_u32(smem + stage * C::STAGE);
                        const uint64_t dx = tc::make_smem_desc_sw128(ax);
                        const uint64_t dy = tc::make_smem_desc_sw128(ax + C::STAGE_X);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // +32 bytes per K step inside the 128-byte swizzle row: +2 in 16-byte units
                            tc::umma_bf16(tmem_d, dx + 2 * k, dy + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        }
                        tc::umma_commit(&empty[stage]);
                        if (++stage == n_stages) { stage = 0; phase ^= 1; }
                    }
                    if (ok) tc::umma_commit(&acc_full[acc]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;  // the TMEM lanes this warp may read: [32*quarter, +32)
        pdl_wait();  // the output may be memory that the previous kernel still reads
        uint32_t local = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++local) {
            const int s = (int)(w % p.n_split);
            const long long rest = w / p.n_split;
            const int tx = (int)(rest % p.tiles_x), ty = (int)(rest / p.tiles_x);
            const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
            if (!tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { if (threadIdx.x == 64) report(p.error, 4, (int)w, -1, (int)acc, MODE, BN); ok = false; break; }
            tc::fence_after_sync();
            const int i = tx * BM + quarter * 32 + lane;  // row of X
            TO* out = reinterpret_cast<TO*>(p.out) + (size_t)s * p.split_stride;
            constexpr int CH = (BN >= 32) ? 32 : 16;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * C::ACC_W + c0;
                if (DUAL) {
                    // h = gate * sigmoid(gate) * up (infer/forward.odin:128-133), both halves from TMEM
                    uint32_t u[32];
                    tc::tmem_ld32(taddr, r);
                    tc::tmem_ld32(taddr + BN, u);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 32; ++q) {
                        float g = __uint_as_float(r[q]);
                        g = __fdividef(g, 1.0f + __expf(-g));  // one ex2 and one rcp: the epilogue's arithmetic is not free beside the MMAs
                        r[q] = __float_as_uint(g * __uint_as_float(u[q]));
                    }
                } else if (CH == 32) {
                    tc::tmem_ld32(taddr, r);
                } else {
                    uint32_t r16[16];
                    tc::tmem_ld16(taddr, r16);
#pragma unroll
                    for (int q = 0; q < 16; ++q) r[q] = r16[q];
                }
                tc::tmem_ld_wait();
                const int j0 = ty * BN + c0;  // first row of Y in this chunk
                if (MODE == 0) {
                    // C[i][j0 + c]: each thread writes a run of its own row
                    if (i < p.rows_x && j0 < p.rows_y) {
                        const int n = min(CH, p.rows_y - j0);
                        store_vec<TO>(out + (size_t)i * p.ldc + j0, r, n);
                    }
                } else {
                    // C[j0 + c][i]: the warp writes 32 consecutive elements of one row
                    if (i < p.rows_x) {
#pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            if (j0 + c < p.rows_y) {
                                out[(size_t)(j0 + c) * p.ldc + i] = from_f32<TO>(__uint_as_float(r[c]));
                            }
                        }
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[acc]);
        }
        if (threadIdx.x == 64) odin_trace_mark(5, true);  // the last tile is stored
    }

    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error != nullptr) atomicCAS(p.error, 0, 99);
    if (warp == 1) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, tmem_cols);
    }
}

// A tile of 128 x 64 bfloat16 through TMA into shared memory, from there by tcgen05.cp into tensor memory,
// and back out through tcgen05.ld: out[row][c] must be the row's elements 2c and 2c + 1 (the layout in which
// an MMA reads its A operand from tensor memory).  Checks the copy that stages weights in tensor memory.
__global__ void __launch_bounds__(128, 1)
stage_probe_kernel(const __grid_constant__ CUtensorMap map_x, uint32_t* __restrict__ out, int* error) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + BM * BK * 2);
    uint64_t* done = full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        tc::mbar_init(full, 1);
        tc::mbar_init(done, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, 32);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        tc::mbar_expect_tx(full, BM * BK * 2);
        tc::tma_load_2d(smem, &map_x, 0, 0, full);
        if (tc::mbar_wait(full, 0, abort_flag)) {
            tc::fence_after_sync();
            const uint64_t dx = tc::make_smem_desc_sw128(tc::smem_u32(smem));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) tc::tmem_cp_128x256b(tmem_base + 8 * k, dx + 2 * k);
        }
        tc::umma_commit(done);
    }
    const bool ok = tc::mbar_wait(done, 0, abort_flag);
    tc::fence_after_sync();
    if (ok) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16), r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) out[(size_t)(warp * 32 + lane) * 32 + c] = r[c];
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && error != nullptr) atomicCAS(error, 0, 98);
    if (warp == 0) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, 32);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    long long rows, K, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ std::hash<long long>()(k.rows);
        h = h * 1000003u ^ std::hash<long long>()(k.K);
        h = h * 1000003u ^ std::hash<long long>()(k.ld);
        return h * 1000003u ^ (size_t)k.box_rows;
    }
};

// A row-major [rows, K] bfloat16 matrix with row stride ld, read in boxes of
// 64 (K) x box_rows, 128-byte swizzle, zeros beyond the edges.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, K, ld, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return ODIN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ODIN_ERR_BAD_ARG;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

// The same matrix seen as [K / 64 blocks][rows][64]: a box of `blocks` K blocks of box_rows x 64 lands as that many
// swizzled tiles one after the other.  K must be a multiple of 64 (else the last block would run into the next row).
int make_map3(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows, int blocks) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, K, ld, box_rows * 1024 + blocks};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return ODIN_ERR_UNSUPPORTED;
    cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, (cuuint64_t)(K / BK)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)BK * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)blocks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ODIN_ERR_BAD_ARG;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

int* error_flag() {
    static int* flag = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&flag, 8 * sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, 8 * sizeof(int));
        else flag = nullptr;
    });
    return flag;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

template <int BN, int MODE, typename TO, bool DUAL = false>
int launch(const CUtensorMap& mx, const CUtensorMap& my, const GemmParams& p, cudaStream_t s,
           const void* y_ptr = nullptr, long long y_ld = 0) {
    using C = Cfg<BN, DUAL>;
    auto kern = gemm_tc_kernel<BN, MODE, TO, DUAL>;
    constexpr int MOST_SMEM = 227 * 1024;  // what a CTA may ask for at all
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             MODE == 1 ? MOST_SMEM : C::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long items = (long long)p.tiles_x * p.tiles_y * p.n_split;
    const int grid = (int)(items < sm_count() ? items : sm_count());
    GemmParams q = p;
    q.stages = (p.stages >= 2 && p.stages < C::STAGES) ? p.stages : C::STAGES;
    // staged blocks: as many as asked for, as tensor memory has columns for beside the accumulators, and as
    // shared memory has room for their token tiles
    q.staged = 0;
    if (MODE == 1 && !DUAL && p.staged > 0) {
        const int by_tmem = (512 - ACC_BUFS * C::ACC_W) / 32;
        const int by_smem = (MOST_SMEM - (C::SMEM - (C::STAGES - q.stages) * C::STAGE)) / C::STAGE_Y1;
        q.staged = p.staged < by_tmem ? p.staged : by_tmem;
        if (q.staged > by_smem) q.staged = by_smem;
        if (q.staged < 0 || y_ptr == nullptr || (p.K % BK) != 0) q.staged = 0;  // the staged tokens' tiles come as one box of whole K blocks
    }
    CUtensorMap my3 = my;
    if (q.staged > 0) {
        int rc = make_map3(&my3, y_ptr, p.rows_y, p.K, y_ld, BN, q.staged);
        if (rc) return rc;
    }
    size_t smem = (size_t)C::SMEM - (size_t)(C::STAGES - q.stages) * C::STAGE + (size_t)q.staged * C::STAGE_Y1;
    // A CTA with staged weights holds all of tensor memory; a second one on the same SM would sit in its
    // allocation until the first is gone instead of fetching weights (measured: the step 14 % slower).  It asks
    // for more than half of an SM's shared memory, so no two of them ever share an SM.
    if (q.staged > 0 && smem < (size_t)117 * 1024) smem = (size_t)117 * 1024;
    odin_launch(kern, dim3(grid), dim3(192), smem, s, mx, my, my3, q);
    ODIN_LAUNCH_CHECK();
    return 0;
}

template <int MODE, typename TO>
int dispatch_bn(int bn, const CUtensorMap& mx, const CUtensorMap& my, const GemmParams& p, cudaStream_t s,
                const void* y_ptr = nullptr, long long y_ld = 0) {
    switch (bn) {
        case 16: return launch<16, MODE, TO>(mx, my, p, s, y_ptr, y_ld);
        case 32: return launch<32, MODE, TO>(mx, my, p, s, y_ptr, y_ld);
        case 64: return launch<64, MODE, TO>(mx, my, p, s, y_ptr, y_ld);
        case 128: return launch<128, MODE, TO>(mx, my, p, s, y_ptr, y_ld);
        case 256: return launch<256, MODE, TO>(mx, my, p, s, y_ptr, y_ld);
        default: return ODIN_ERR_UNSUPPORTED;
    }
}

}  // namespace

// A: [M, K] bfloat16, row stride lda; W: [N, K] bfloat16, row stride ldw; C: [M, N] of
// c_dtype, row stride ldc, or with n_split > 1: float32 partial sums [n_split][M][ldc...]
// split_stride elements apart.  mode 0: tokens on the 128-row side; mode 1: weights on
// it (for M <= bn).  bn: the tile's N side: 16..256.  Strides and K must be multiples
// of 8 elements and the pointers 16-byte aligned (TMA), else ODIN_ERR_UNSUPPORTED.
// stages: the length of the ring of shared-memory stages; 0: as many as fit (the product then has the SM to
// itself), fewer to let a CTA of the kernel before or after it share the SM.
// staged (mode 1): K blocks of each CTA's first item whose weights wait in tensor memory while the kernel before
// this one still runs (fewer where tensor or shared memory has no room for them); the result is the same bits.
extern "C" int odin_gemm_tc(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, long long lda,
                            long long ldw, long long ldc, int mode, int bn, int n_split, long long split_stride,
                            int stages, int staged, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || n_split < 1) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    if (n_split > 1 && c_dtype != ODIN_F32) return ODIN_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    GemmParams p;
    p.out = C;
    p.ldc = ldc;
    p.split_stride = split_stride;
    p.K = K;
    p.kb_total = (K + BK - 1) / BK;
    if (n_split > p.kb_total) n_split = p.kb_total;
    p.kb_per_split = (p.kb_total + n_split - 1) / n_split;
    if ((p.kb_total + p.kb_per_split - 1) / p.kb_per_split != n_split) return ODIN_ERR_BAD_ARG;  // an empty part
    p.n_split = n_split;
    p.dual_offset = 0;
    p.stages = stages;
    p.staged = mode == 1 ? staged : 0;
    p.error = error_flag();
    CUtensorMap mx, my;
    int rc;
    if (mode == 0) {
        p.rows_x = M; p.rows_y = N;
        if ((rc = make_map(&mx, A, M, K, lda, BM))) return rc;
        if ((rc = make_map(&my, W, N, K, ldw, bn))) return rc;
    } else if (mode == 1) {
        p.rows_x = N; p.rows_y = M;
        if ((rc = make_map(&mx, W, N, K, ldw, BM))) return rc;
        if ((rc = make_map(&my, A, M, K, lda, bn))) return rc;
    } else {
        return ODIN_ERR_BAD_ARG;
    }
    p.tiles_x = (p.rows_x + BM - 1) / BM;
    p.tiles_y = (p.rows_y + bn - 1) / bn;
    if (c_dtype == ODIN_F32)
        return mode == 0 ? dispatch_bn<0, float>(bn, mx, my, p, s) : dispatch_bn<1, float>(bn, mx, my, p, s, A, lda);
    if (c_dtype == ODIN_BF16)
        return mode == 0 ? dispatch_bn<0, bf16>(bn, mx, my, p, s) : dispatch_bn<1, bf16>(bn, mx, my, p, s, A, lda);
    return ODIN_ERR_UNSUPPORTED;
}

// C[M, I] = silu(A Wg^T) * (A Wu^T) for W = [Wg; Wu] of shape [2 I, K]: the gate and up products
// accumulate side by side in tensor memory and the SwiGLU is applied as they are read back, so
// the [M, 2 I] intermediate never exists.  For many tokens (mode 0, tiles of 128 output columns).
extern "C" int odin_gemm_tc_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int I, int K,
                                   long long lda, long long ldw, long long ldc, void* stream) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    constexpr int BN = 128;
    GemmParams p;
    p.out = C;
    p.ldc = ldc;
    p.split_stride = 0;
    p.K = K;
    p.kb_total = (K + BK - 1) / BK;
    p.kb_per_split = p.kb_total;
    p.n_split = 1;
    p.stages = 0;
    p.staged = 0;
    p.dual_offset = I;
    p.error = error_flag();
    p.rows_x = M;
    p.rows_y = I;
    CUtensorMap mx, my;
    int rc;
    if ((rc = make_map(&mx, A, M, K, lda, BM))) return rc;
    if ((rc = make_map(&my, W, 2LL * I, K, ldw, BN))) return rc;
    p.tiles_x = (M + BM - 1) / BM;
    p.tiles_y = (I + BN - 1) / BN;
    cudaStream_t s = (cudaStream_t)stream;
    if (c_dtype == ODIN_BF16) return launch<BN, 0, bf16, true>(mx, my, p, s);
    if (c_dtype == ODIN_F32) return launch<BN, 0, float, true>(mx, my, p, s);
    return ODIN_ERR_UNSUPPORTED;
}

// X: [128, 64] bfloat16, contiguous; out: [128, 32] 32-bit words (see stage_probe_kernel).
extern "C" int odin_gemm_tc_stage_probe(const void* X, void* out, void* stream) {
    if ((((uintptr_t)X) & 15) != 0) return ODIN_ERR_UNSUPPORTED;
    CUtensorMap mx;
    int rc;
    if ((rc = make_map(&mx, X, BM, BK, BK, BM))) return rc;
    const size_t smem = BM * BK * 2 + 1024 + 64;
    stage_probe_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(mx, (uint32_t*)out, error_flag());
    ODIN_LAUNCH_CHECK();
    return 0;
}

// The number of K parts that odin_gemm_tc will really use for (K, n_split).
extern "C" int odin_gemm_tc_splits(int K, int n_split) {
    const int kb_total = (K + BK - 1) / BK;
    if (n_split > kb_total) n_split = kb_total;
    if (n_split < 1) n_split = 1;
    const int per = (kb_total + n_split - 1) / n_split;
    return (kb_total + per - 1) / per;
}

// Reads and clears the flag that a kernel sets when one of its bounded waits ran
// out (synchronises the device).  0: all well.
extern "C" int odin_gemm_tc_error() {
    int* f = error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(f, 0, sizeof(int));
    return v;
}

// The same, with the details of the first wait that ran out (8 ints, see `report`); does not clear.
extern "C" int odin_gemm_tc_error_detail(int* out8) {
    int* f = error_flag();
    if (f == nullptr) return 0;
    if (cudaMemcpy(out8, f, 8 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return out8[0];
}

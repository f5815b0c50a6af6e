// A decode step of few tokens as a program: a short list of operations that ONE persistent
// kernel (a CTA per SM) carries out one after the other, with a barrier across the grid
// between two of them instead of a kernel boundary.
//
// Why: a decode step is a chain of small kernels, each bound by the weights it streams from
// memory.  Between two kernels the memory system idles for microseconds: the last tiles'
// products, the epilogue, the grid's completion, the next kernel's start and its first loads.
// Here the warp that requests weight tiles never stops: weights depend on nothing, so while
// the other warps finish one operation, meet at the barrier and run a small operation (a
// norm, attention over the cache), it already fills the ring of stages with the next
// product's weights.
//
// Operations: a matrix product of few tokens (weights on the 128-row side of tcgen05.mma,
// tokens on its N side, split along K, 32-bit partial sums out: gemm_tc.cu's mode 1),
// residual add + RMSNorm (elementwise.cu), SwiGLU of partial sums (elementwise.cu), and
// decode attention with head preparation (attention_decode_tc.cuh).  The products, the SwiGLU
// and attention add in the same order as the kernels of their own; the norm is spread over all
// CTAs (pieces of 512 columns, their sums of squares met across the grid), so its sum of squares
// is added up in another order.
//
// Measured (8B layer sizes, 8 sequences): the products stream their weights faster this way (65
// against 77 us per layer, boundaries included), but the operations between them no longer overlap
// the products' ends as co-resident kernels do, a barrier costs 2 to 3 us, and a layer takes 120 us
// against 95.  The runtime therefore uses it only on request.
//
// Roles (256 threads): warp 0 requests weight tiles (TMA), warp 1 requests activation tiles
// (TMA; it is the one that waits for the operation before), warp 2 issues the MMAs, warp 3
// rests, warps 4..7 are the workers: they read accumulators back and run the other
// operations.  A stage's barrier takes two arrivals, one from each requesting warp.
//
// The barrier across the grid: one counter per operation; the workers of a CTA add one when
// they have finished it (a release), and whoever needs its result waits until the counter
// has reached the number of CTAs (an acquire; before TMA reads it, a proxy fence).  All CTAs are resident at once (one per SM, never
// more CTAs than SMs).  Every wait has a limit, after which the kernel sets the error flag
// and leaves.  The CTA that leaves last clears the counters for the next launch.
//
// In the reference the step is the loop over layers of infer/forward.odin:40-143.
#include <mutex>

#include "attention_decode_tc.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int ACC_BUFS = 2;
constexpr int MAX_OPS = 8;
constexpr int MAX_MAPS = 10;
constexpr int MAX_STAGES = 12;
constexpr int ATTN_SLOTS = 3;
constexpr int NORM_PIECE = 512;     // columns of a row that one CTA takes at a time (a float4 per worker thread)
constexpr int NORM_MAX_PIECES = 4;  // pieces per CTA: their sums stay in registers across the barrier
constexpr int NORM_SSQ_FLOATS = 2048;  // scratch per operation

enum { OP_GEMM = 1, OP_ADDNORM = 2, OP_SWIGLU = 3, OP_ATTN = 4 };

struct GemmOp {
    float* out;  // [n_split][rows_y][ldc...] partial sums
    long long ldc, split_stride;
    int rows_x, rows_y, tiles_x, n_split, kb_per_split, kb_total;
    int map;     // the weight's tensor map; the activations' is the next one
};
struct NormOp {  // x += sum of delta's parts; out = RMSNorm(x) * w
    float* ssq;  // [n_rows][d / 512] scratch: each 512-column piece's share of its row's sum of squares
    float* x;
    const float* delta;  // [n_split][n_rows][d], or null
    long long split_stride;
    int n_split;
    VecRef w;
    float eps;
    bf16* out;
    int n_rows, d;
};
struct SwigluOp {  // out[t][j] = silu(sum gate) * (sum up)
    const float* gu;  // [n_split][T][2 I]
    long long split_stride;
    int n_split;
    bf16* out;
    int T, I;
};
struct AttnOp {  // the attention's own parameters are Program::attn: a program holds one attention at most
    int map;     // K's tensor map; V's is the next one
    int B;
};
struct ProgOp {
    int kind;
    union {
        GemmOp g;
        NormOp n;
        SwigluOp s;
        AttnOp a;
    };
};
struct Program {
    CUtensorMap maps[MAX_MAPS];
    ProgOp ops[MAX_OPS];
    // The one attention's parameters, apart from the operations: at a fixed place among the kernel's
    // parameters they are read as constants, where a copy in shared memory costs the attention loop
    // the registers that it does not have.
    attn_decode::DecodeTcParams attn;
    int n_ops;
    int n_stages;
    int* sync;   // [0]: CTAs that have left; [1 + j]: CTAs that have finished operation j;
                 // [1 + MAX_OPS + j]: CTAs that have finished the first half of operation j (a norm)
    int* error;  // [0] set when a wait ran out, [1..7] who it was
};
static_assert(sizeof(Program) <= 4096, "the program travels as a kernel parameter");

template <int BN, int HD>
struct PCfg {
    static constexpr int STAGE_X = BM * BK * 2;
    static constexpr int STAGE_Y = BN * BK * 2;
    static constexpr int STAGE = STAGE_X + STAGE_Y;
    static constexpr int ATTN = HD > 0 ? attn_decode::DecodeTcSmem<(HD > 0 ? HD : 64), ATTN_SLOTS>::BYTES - 1024 : 0;
    static constexpr int ATTN_PAD = (ATTN + 1023) / 1024 * 1024;
    static constexpr int TAIL = 3072;  // barriers, flags, the norm's reduction; the operations
    static constexpr int BUDGET = 232448 - 1024 /*alignment*/ - TAIL - ATTN_PAD;
    static constexpr int STAGES = (BUDGET / STAGE) > MAX_STAGES ? MAX_STAGES : (BUDGET / STAGE);
    static constexpr int TMEM_COLS = (ACC_BUFS * BN) < 32 ? 32 : (ACC_BUFS * BN);
    static constexpr int smem(int stages) { return stages * STAGE + ATTN_PAD + TAIL + 1024; }
};

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Orders this thread's earlier accesses to global memory through the ordinary path (here: the acquire
// that saw other CTAs' stores) before its later ones through the asynchronous path (TMA loads).
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

__device__ __noinline__ void report(int* err, int what, int op, int item, int kb, int slot) {
    if (err == nullptr) return;
    if (atomicCAS(err, 0, what) == 0) {
        err[1] = (int)blockIdx.x; err[2] = op; err[3] = item; err[4] = kb; err[5] = slot; err[6] = (int)gridDim.x;
    }
}

// Has every CTA finished the operation whose counter this is?  One thread asks; it must fence (or
// meet the others at a barrier) before anyone reads what the operation wrote.
__device__ __forceinline__ bool grid_wait(const int* counter, int target, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t n = 1;; ++n) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) return true;
        if (*abort_flag) return false;
        if ((n & 63) == 0) {
            const unsigned long long now = tc::global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > TC_WAIT_SECONDS * 1000000000ull) { *abort_flag = 1; return false; }
        }
        __nanosleep(20);
    }
}

// The operations of the workers (128 threads, wt = 0..127), each a function of its own so that its
// registers are its own.  wait_before(): called by all of them together where the operation first
// needs what ran before it.
// Residual add + RMSNorm over all CTAs: the rows are cut into pieces of 512 columns, a piece per CTA
// at a time and a float4 per thread, so that all loads of the operation are in flight at once.  Each
// piece's share of its row's sum of squares goes to scratch; after a barrier across the grid every
// piece adds up its row's shares (in the order of the pieces: the same whatever else is in the batch)
// and writes its normed columns from the sums that it kept in registers.
template <typename WaitFn>
__device__ __noinline__ void run_norm(const NormOp& n, const int wt, const int lane, const int quarter, const int grid,
                                      float* s_red, const int* half_counter, volatile int* abort_flag, int* error,
                                      const int j, WaitFn& wait_before) {
    const int per_row = (n.d + NORM_PIECE - 1) / NORM_PIECE;  // the last piece of a row may be short
    const int row_v = n.d / 4;                                // float4 per row
    const int n_pieces = n.n_rows * per_row;
    float4 v[NORM_MAX_PIECES], wv[NORM_MAX_PIECES];
    // the weights depend on nothing: fetched ahead of the wait
#pragma unroll
    for (int k = 0; k < NORM_MAX_PIECES; ++k) {
        const int piece = (int)blockIdx.x + k * grid;
        const int c = (piece % per_row) * (NORM_PIECE / 4) + wt;  // float4 within the row
        if (piece < n_pieces && c < row_v) {
            if (n.w.is_bf16) {
                const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(n.w.p) + 4 * c);
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
                wv[k] = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
            } else {
                wv[k] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(n.w.p) + 4 * c);
            }
        }
    }
    wait_before();
#pragma unroll
    for (int k = 0; k < NORM_MAX_PIECES; ++k) {
        const int piece = (int)blockIdx.x + k * grid;
        if (piece < n_pieces) {  // the same for all workers of the CTA
            const int r = piece / per_row, c = (piece % per_row) * (NORM_PIECE / 4) + wt;
            const bool on = c < row_v;
            float4* xr = reinterpret_cast<float4*>(n.x + (size_t)r * n.d) + c;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on) acc = __ldcg(xr);
            if (on && n.delta != nullptr) {
                const float4* dp = reinterpret_cast<const float4*>(n.delta + (size_t)r * n.d) + c;
                for (int s0 = 0; s0 < n.n_split; s0 += 4) {  // x, then the parts in order
                    float4 d[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (s0 + u < n.n_split) d[u] = __ldcg(dp + (size_t)(s0 + u) * (n.split_stride / 4));
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (s0 + u < n.n_split) { acc.x += d[u].x; acc.y += d[u].y; acc.z += d[u].z; acc.w += d[u].w; }
                }
                *xr = acc;
            }
            v[k] = acc;
            float ss = 0.f;
            ss += acc.x * acc.x; ss += acc.y * acc.y; ss += acc.z * acc.z; ss += acc.w * acc.w;
            ss = warp_sum(ss);
            if (lane == 0) s_red[quarter] = ss;
            workers_sync();
            if (wt == 0) n.ssq[piece] = ((s_red[0] + s_red[1]) + s_red[2]) + s_red[3];
            workers_sync();  // s_red is free for the next piece
        }
    }
    // the shares meet
    workers_sync();
    if (wt == 0) {
        asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(half_counter) : "memory");
        if (!grid_wait(half_counter, grid, abort_flag)) report(error, 8, j, -1, -1, -1);
    }
    workers_sync();
#pragma unroll
    for (int k = 0; k < NORM_MAX_PIECES; ++k) {
        const int piece = (int)blockIdx.x + k * grid;
        if (piece < n_pieces) {
            const int r = piece / per_row, c = (piece % per_row) * (NORM_PIECE / 4) + wt;
            if (c >= row_v) continue;
            const float* shares = n.ssq + (size_t)r * per_row;
            float ss = 0.f;
            for (int q0 = 0; q0 < per_row; q0 += 8) {
                float sh[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) sh[u] = (q0 + u < per_row) ? __ldcg(shares + q0 + u) : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u) ss += sh[u];
            }
            ss /= (float)n.d;
            ss += n.eps;
            const float rs = 1.0f / sqrtf(ss);
            uint2 u2;
            u2.x = attn::pack_bf16(wv[k].x * (rs * v[k].x), wv[k].y * (rs * v[k].y));
            u2.y = attn::pack_bf16(wv[k].z * (rs * v[k].z), wv[k].w * (rs * v[k].w));
            reinterpret_cast<uint2*>(n.out + (size_t)r * n.d)[c] = u2;
        }
    }
}

template <typename WaitFn>
__device__ __noinline__ void run_swiglu(const SwigluOp& sw, const int wt, const int grid, WaitFn& wait_before) {
    wait_before();
    const int I4 = sw.I / 4;
    const int total4 = sw.T * I4;
    for (int idx = blockIdx.x * 128 + wt; idx < total4; idx += grid * 128) {
        const int t = idx / I4;
        const int c = (idx - t * I4) * 4;
        const float* row = sw.gu + (size_t)t * 2 * sw.I + c;
        float4 gsum = make_float4(0.f, 0.f, 0.f, 0.f), usum = gsum;
        for (int s0 = 0; s0 < sw.n_split; s0 += 4) {
            float4 gv[4], uv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                if (s0 + a < sw.n_split) {
                    gv[a] = __ldcg(reinterpret_cast<const float4*>(row + (size_t)(s0 + a) * sw.split_stride));
                    uv[a] = __ldcg(reinterpret_cast<const float4*>(row + (size_t)(s0 + a) * sw.split_stride + sw.I));
                }
            }
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                if (s0 + a < sw.n_split) {
                    gsum.x += gv[a].x; gsum.y += gv[a].y; gsum.z += gv[a].z; gsum.w += gv[a].w;
                    usum.x += uv[a].x; usum.y += uv[a].y; usum.z += uv[a].z; usum.w += uv[a].w;
                }
            }
        }
        // h = g * (1 / (1 + exp(-g))) * u in that order of products (infer/forward.odin:128-133)
        gsum.x *= 1.0f / (1.0f + expf(-gsum.x)); gsum.x *= usum.x;
        gsum.y *= 1.0f / (1.0f + expf(-gsum.y)); gsum.y *= usum.y;
        gsum.z *= 1.0f / (1.0f + expf(-gsum.z)); gsum.z *= usum.z;
        gsum.w *= 1.0f / (1.0f + expf(-gsum.w)); gsum.w *= usum.w;
        uint2 u;
        u.x = attn::pack_bf16(gsum.x, gsum.y);
        u.y = attn::pack_bf16(gsum.z, gsum.w);
        *reinterpret_cast<uint2*>(sw.out + (size_t)t * sw.I + c) = u;
    }
}

template <int HD, typename WaitFn>
__device__ __forceinline__ void run_attention(const Program& P, const AttnOp& a, uint8_t* attn_smem, const int wt,
                                              const int grid, WaitFn& wait_before) {
    const attn_decode::DecodeTcParams& p = P.attn;
    const int n_items = p.n_split * p.Hkv * a.B;
    bool waited = false;
    auto wait_once = [&]() {
        if (!waited) { wait_before(); waited = true; }
    };
    for (int w = blockIdx.x; w < n_items; w += grid) {
        const int split = w % p.n_split, rest = w / p.n_split;
        attn_decode::attn_decode_tc_body<HD, ATTN_SLOTS, 1, 1>(P.maps[a.map], P.maps[a.map + 1], p, attn_smem, wt, split,
                                                               rest % p.Hkv, rest / p.Hkv, wait_once);
        workers_sync();  // the shared memory is free for the next piece
    }
    wait_once();
}

template <int BN, int HD>
__global__ void __launch_bounds__(256, 1) decode_program_kernel(const __grid_constant__ Program P) {
    using C = PCfg<BN, HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t n_stages = (uint32_t)P.n_stages;
    uint8_t* attn_smem = smem + n_stages * C::STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(attn_smem + C::ATTN_PAD);
    uint64_t* full = bars;                                // [MAX_STAGES] both tiles landed
    uint64_t* empty = bars + MAX_STAGES;                  // [MAX_STAGES] the MMAs that read the stage are done
    uint64_t* acc_full = bars + 2 * MAX_STAGES;           // [ACC_BUFS]
    uint64_t* acc_empty = acc_full + ACC_BUFS;            // [ACC_BUFS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* s_red = reinterpret_cast<float*>(tmem_slot + 4);  // [8] the norm's reduction
    // The operations, copied from the parameters: indexed by a variable there they would be copied to
    // every thread's local memory instead.
    ProgOp* s_ops = reinterpret_cast<ProgOp*>(reinterpret_cast<uint8_t*>(bars) + 512);
    static_assert(512 + sizeof(ProgOp) * MAX_OPS <= C::TAIL, "the operations do not fit");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = (int)gridDim.x;
    const int n_ops = P.n_ops;
    pdl_trigger();

#pragma unroll
    for (int j = 0; j < MAX_OPS; ++j)
        if ((int)threadIdx.x == 32 + j && j < P.n_ops) s_ops[j] = P.ops[j];
    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            tc::mbar_init(&full[s], 2);  // one arrival from each requesting warp
            tc::mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < ACC_BUFS; ++a) {
            tc::mbar_init(&acc_full[a], 1);
            tc::mbar_init(&acc_empty[a], 4);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    if (warp == 2) tc::tmem_alloc(tmem_slot, C::TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------ weight tiles: never waits for an operation
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int j = 0; j < n_ops && ok; ++j) {
                if (s_ops[j].kind != OP_GEMM) continue;
                const GemmOp& g = s_ops[j].g;
                const CUtensorMap* map_w = &P.maps[g.map];
                const int n_items = g.tiles_x * g.n_split;
                for (int w = blockIdx.x; w < n_items && ok; w += grid) {
                    const int s = w % g.n_split, tx = w / g.n_split;
                    const int kb0 = s * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report(P.error, 1, j, w, kb, stage); ok = false; break; }
                        tc::mbar_expect_tx(&full[stage], C::STAGE_X);
                        tc::tma_load_2d(smem + stage * C::STAGE, map_w, kb * BK, tx * BM, &full[stage]);
                        if (++stage == n_stages) { stage = 0; phase ^= 1; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ activation tiles: waits for the operation before
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            pdl_wait();  // the counters, too, are the launch before's until it is over
            for (int j = 0; j < n_ops && ok; ++j) {
                if (s_ops[j].kind != OP_GEMM) continue;
                const GemmOp& g = s_ops[j].g;
                const CUtensorMap* map_y = &P.maps[g.map + 1];
                const int n_items = g.tiles_x * g.n_split;
                if ((int)blockIdx.x >= n_items) continue;
                if (j > 0 && !grid_wait(P.sync + 1 + (j - 1), grid, abort_flag)) { report(P.error, 5, j, -1, -1, -1); ok = false; break; }
                fence_proxy_async_global();  // other CTAs' ordinary stores, now read by TMA
                for (int w = blockIdx.x; w < n_items && ok; w += grid) {
                    const int s = w % g.n_split;
                    const int kb0 = s * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report(P.error, 2, j, w, kb, stage); ok = false; break; }
                        tc::mbar_expect_tx(&full[stage], C::STAGE_Y);
                        tc::tma_load_2d(smem + stage * C::STAGE + C::STAGE_X, map_y, kb * BK, 0, &full[stage]);
                        if (++stage == n_stages) { stage = 0; phase ^= 1; }
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------ MMA issuer: the warp walks converged, one lane issues
        constexpr uint32_t idesc = tc::make_idesc_bf16(BM, BN);
        uint32_t stage = 0, phase = 0, local = 0;
        bool ok = true, ready = false;
        for (int j = 0; j < n_ops && ok; ++j) {
            if (s_ops[j].kind != OP_GEMM) continue;
            const GemmOp& g = s_ops[j].g;
            const int n_items = g.tiles_x * g.n_split;
            for (int w = blockIdx.x; w < n_items && ok; w += grid, ++local) {
                const int s = w % g.n_split;
                const int kb0 = s * g.kb_per_split, kb1 = min(g.kb_total, kb0 + g.kb_per_split);
                const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
                ok = __all_sync(0xffffffffu, tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag));
                if (!ok) { if (lane == 0) report(P.error, 3, j, w, -1, (int)acc); break; }
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!ready) ready = tc::mbar_wait(&full[stage], phase, abort_flag);
                    ok = __all_sync(0xffffffffu, ready);
                    if (!ok) { if (lane == 0) report(P.error, 4, j, w, kb, stage); break; }
                    tc::fence_after_sync();
                    const uint32_t cur = stage;
                    if (++stage == n_stages) { stage = 0; phase ^= 1; }
                    ready = __all_sync(0xffffffffu, tc::mbar_test_wait(&full[stage], phase));
                    if (tc::elect_one()) {
                        const uint32_t ax = tc::smem_u32(smem + cur * C::STAGE);
                        const uint64_t dx = tc::make_smem_desc_sw128(ax);
                        const uint64_t dy = tc::make_smem_desc_sw128(ax + C::STAGE_X);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tc::umma_bf16(tmem_d, dx + 2 * k, dy + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        tc::umma_commit(&empty[cur]);
                    }
                    __syncwarp();
                }
                if (ok && tc::elect_one()) tc::umma_commit(&acc_full[acc]);
                __syncwarp();
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------ workers
        const int wt = (int)threadIdx.x - 128;  // 0..127
        const int quarter = warp & 3;           // the TMEM lanes this warp may read
        uint32_t local = 0;
        bool ok = true;
        for (int j = 0; j < n_ops && ok; ++j) {
            const ProgOp& op = s_ops[j];
            // Everything but a product's epilogue starts by waiting for the operation before (a
            // product's epilogue follows its MMAs, whose activations waited): this also keeps an
            // operation's stores behind every reader of memory that the allocator hands out again.
            auto wait_before = [&]() {
                if (j == 0) {
                    pdl_wait();
                } else {
                    if (wt == 0 && !grid_wait(P.sync + 1 + (j - 1), grid, abort_flag)) report(P.error, 6, j, -1, -1, -1);
                    workers_sync();  // the one thread's acquire, handed on to the others
                }
            };
            if (op.kind == OP_GEMM) {
                const GemmOp& g = op.g;
                const int n_items = g.tiles_x * g.n_split;
                if (j == 0) pdl_wait();  // also a CTA without a tile counts itself only after the launch before is over
                for (int w = blockIdx.x; w < n_items && ok; w += grid, ++local) {
                    const int s = w % g.n_split, tx = w / g.n_split;
                    const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
                    if (!tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { if (wt == 0) report(P.error, 7, j, w, -1, (int)acc); ok = false; break; }
                    tc::fence_after_sync();
                    const int i = tx * BM + quarter * 32 + lane;  // row of the weight: column of the output
                    float* out = g.out + (size_t)s * g.split_stride;
                    constexpr int CH = (BN >= 32) ? 32 : 16;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += CH) {
                        if (c0 >= g.rows_y) break;
                        uint32_t r[CH];
                        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0;
                        if constexpr (CH == 32) tc::tmem_ld32(taddr, r);
                        else tc::tmem_ld16(taddr, r);
                        tc::tmem_ld_wait();
                        if (i < g.rows_x) {
#pragma unroll
                            for (int c = 0; c < CH; ++c)
                                if (c0 + c < g.rows_y) out[(size_t)(c0 + c) * g.ldc + i] = __uint_as_float(r[c]);
                        }
                    }
                    tc::fence_before_sync();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[acc]);
                }
            } else if (op.kind == OP_ADDNORM) {
                run_norm(op.n, wt, lane, quarter, grid, s_red, P.sync + 1 + MAX_OPS + j, abort_flag, P.error, j, wait_before);
            } else if (op.kind == OP_SWIGLU) {
                run_swiglu(op.s, wt, grid, wait_before);
            } else if (op.kind == OP_ATTN) {
                if constexpr (HD > 0) {
                    run_attention<HD>(P, op.a, attn_smem, wt, grid, wait_before);
                }
            }
            // the operation is done here: make its stores visible (to TMA too) and count this CTA
            workers_sync();  // all workers' stores are ordered before the one thread's release
            if (wt == 0) {
                asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(P.sync + 1 + j) : "memory");
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: copies may still be in flight; give them time to land before the shared memory is released
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (*abort_flag && P.error != nullptr) atomicCAS(P.error, 0, 99);
        __threadfence();
        if (atomicAdd(P.sync, 1) == grid - 1) {  // the last CTA out: nobody waits on a counter any more
            for (int j = 0; j <= 2 * MAX_OPS; ++j) P.sync[j] = 0;
            __threadfence();
        }
    }
    if (warp == 2) {
        tc::fence_after_sync();
        tc::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
static __device__ int g_prog_error[8];
static __device__ int g_prog_sync[2 * MAX_OPS + 1];
static __device__ float g_prog_ssq[MAX_OPS * NORM_SSQ_FLOATS];
constexpr int PROG_SPLIT_COUNTERS = 1 << 14;
static __device__ int g_prog_split_counters[PROG_SPLIT_COUNTERS];

template <typename T>
int* device_symbol(const T& symbol, int which) {
    constexpr int MAX_DEVICES = 64;
    static int* addr[4][MAX_DEVICES] = {{nullptr}};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> g(mu);
    if (addr[which][dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, symbol) != cudaSuccess) return nullptr;
        addr[which][dev] = static_cast<int*>(p);
    }
    return addr[which][dev];
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// A row-major [rows, K] bfloat16 matrix with row stride ld, read in boxes of 64 (K) x box_rows,
// 128-byte swizzle, zeros beyond the edges.
int matrix_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    attn::EncodeTiledFn fn = attn::encode_fn();
    if (fn == nullptr) return ODIN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ODIN_ERR_BAD_ARG;
}

// The program being recorded (one per process; recording and running are the caller's single thread's).
struct Builder {
    bool open = false;
    int bn = 0, hd = 0;
    int n_maps = 0;
    Program prog;
    long long launches = 0;
};
Builder g_builder;

template <int BN, int HD>
int launch_program(Program& prog, cudaStream_t s) {
    using C = PCfg<BN, HD>;
    static_assert(C::STAGES >= 2, "no room for a ring of stages");
    auto kern = decode_program_kernel<BN, HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smem(C::STAGES));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    prog.n_stages = C::STAGES;
    odin_launch(kern, dim3(sm_count()), dim3(256), (size_t)C::smem(C::STAGES), s, prog);
    ODIN_LAUNCH_CHECK();
    return 0;
}

int run_builder(cudaStream_t s) {
    Builder& b = g_builder;
    if (b.prog.n_ops == 0) return 0;
    b.prog.sync = device_symbol(g_prog_sync, 0);
    b.prog.error = device_symbol(g_prog_error, 1);
    if (b.prog.sync == nullptr || b.prog.error == nullptr) return ODIN_ERR_UNSUPPORTED;
    bool has_attn = false;
    for (int j = 0; j < b.prog.n_ops; ++j) has_attn |= b.prog.ops[j].kind == OP_ATTN;
    int rc = ODIN_ERR_UNSUPPORTED;
#define GO(BN_)                                                                              \
    (!has_attn ? launch_program<BN_, 0>(b.prog, s)                                    \
               : (b.hd == 64 ? launch_program<BN_, 64>(b.prog, s) : launch_program<BN_, 128>(b.prog, s)))
    if (b.bn == 16) rc = GO(16);
    else if (b.bn == 32) rc = GO(32);
    else if (b.bn == 64) rc = GO(64);
#undef GO
    b.prog.n_ops = 0;
    b.n_maps = 0;
    if (rc == 0) ++b.launches;
    return rc;
}

// room for one more operation that needs `maps` tensor maps: a full program is launched first
int make_room(int maps, cudaStream_t s) {
    Builder& b = g_builder;
    if (b.prog.n_ops == MAX_OPS || b.n_maps + maps > MAX_MAPS) return run_builder(s);
    return 0;
}

}  // namespace

// Starts recording a program for steps of at most bn tokens (16, 32 or 64).  Until odin_prog_end the
// odin_prog_* calls below record operations instead of launching kernels; a program that is full is
// launched on the stream given with the call that found it full.  Each returns 0 when the operation
// was recorded, ODIN_ERR_UNSUPPORTED when it cannot be part of a program (the caller then calls
// odin_prog_flush and launches the operation's own kernel), another code for an error.
extern "C" int odin_prog_begin(int bn) {
    if (!(bn == 16 || bn == 32 || bn == 64)) return ODIN_ERR_UNSUPPORTED;
    Builder& b = g_builder;
    if (b.open) return ODIN_ERR_BAD_ARG;
    std::memset(&b.prog, 0, sizeof(b.prog));
    b.open = true; b.bn = bn; b.hd = 0; b.n_maps = 0;
    return 0;
}

// Launches what has been recorded so far; recording goes on.
extern "C" int odin_prog_flush(void* stream) {
    if (!g_builder.open) return 0;
    return run_builder((cudaStream_t)stream);
}

extern "C" int odin_prog_end(void* stream) {
    if (!g_builder.open) return 0;
    const int rc = run_builder((cudaStream_t)stream);
    g_builder.open = false;
    return rc;
}

// Programs launched since the library was loaded.
extern "C" long long odin_prog_launches() { return g_builder.launches; }

// C[n_split][M][N] (32-bit partial sums, slices split_stride elements apart, rows ldc) = A[M, K] W[N, K]^T.
extern "C" int odin_prog_gemm(const void* A, const void* W, float* C, int M, int N, int K, long long lda, long long ldw,
                              long long ldc, int n_split, long long split_stride, void* stream) {
    Builder& b = g_builder;
    if (!b.open) return ODIN_ERR_BAD_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || n_split < 1) return ODIN_ERR_BAD_ARG;
    if (M > b.bn) return ODIN_ERR_UNSUPPORTED;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    GemmOp g;
    g.kb_total = (K + BK - 1) / BK;
    if (n_split > g.kb_total) n_split = g.kb_total;
    g.kb_per_split = (g.kb_total + n_split - 1) / n_split;
    if ((g.kb_total + g.kb_per_split - 1) / g.kb_per_split != n_split) return ODIN_ERR_BAD_ARG;  // an empty part
    if ((long long)((N + BM - 1) / BM) * n_split > (1 << 24)) return ODIN_ERR_UNSUPPORTED;
    int rc = make_room(2, (cudaStream_t)stream);
    if (rc) return rc;
    if ((rc = matrix_map(&b.prog.maps[b.n_maps], W, N, K, ldw, BM))) return rc;
    if ((rc = matrix_map(&b.prog.maps[b.n_maps + 1], A, M, K, lda, b.bn))) return rc;
    g.out = C; g.ldc = ldc; g.split_stride = split_stride;
    g.rows_x = N; g.rows_y = M; g.tiles_x = (N + BM - 1) / BM; g.n_split = n_split;
    g.map = b.n_maps;
    b.n_maps += 2;
    ProgOp& op = b.prog.ops[b.prog.n_ops++];
    op.kind = OP_GEMM;
    op.g = g;
    return 0;
}

// x[n_rows][d] += sum of delta's parts (32-bit, may be null); out = RMSNorm(x) * w in bfloat16.
extern "C" int odin_prog_add_rmsnorm(float* x, const float* delta, int n_split, long long split_stride, const void* w,
                                     int w_dtype, float eps, void* out, int n_rows, int d, void* stream) {
    Builder& b = g_builder;
    if (!b.open) return ODIN_ERR_BAD_ARG;
    if (n_rows <= 0 || d <= 0) return ODIN_ERR_BAD_ARG;
    const long long pieces = (long long)n_rows * ((d + NORM_PIECE - 1) / NORM_PIECE);
    if (n_rows > b.bn || (d % 4) || (split_stride % 4) || pieces > (long long)NORM_MAX_PIECES * sm_count() ||
        pieces > NORM_SSQ_FLOATS ||
        ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)w)) & 15) || (((uintptr_t)out) & 7))
        return ODIN_ERR_UNSUPPORTED;
    int rc = make_room(0, (cudaStream_t)stream);
    if (rc) return rc;
    float* ssq = reinterpret_cast<float*>(device_symbol(g_prog_ssq, 3));
    if (ssq == nullptr) return ODIN_ERR_UNSUPPORTED;
    NormOp n;
    n.ssq = ssq + (size_t)b.prog.n_ops * NORM_SSQ_FLOATS;
    n.x = x; n.delta = delta; n.split_stride = split_stride; n.n_split = delta ? n_split : 0;
    n.w = VecRef{w, w_dtype == ODIN_BF16}; n.eps = eps; n.out = (bf16*)out; n.n_rows = n_rows; n.d = d;
    ProgOp& op = b.prog.ops[b.prog.n_ops++];
    op.kind = OP_ADDNORM;
    op.n = n;
    return 0;
}

// out[T][I] (bfloat16) = silu(gate) * up of the summed parts of gu[n_split][T][2 I] (32-bit).
extern "C" int odin_prog_swiglu(const float* gu, int n_split, long long split_stride, void* out, int T, int I,
                                void* stream) {
    Builder& b = g_builder;
    if (!b.open) return ODIN_ERR_BAD_ARG;
    if (T <= 0 || I <= 0 || n_split < 1) return ODIN_ERR_BAD_ARG;
    if (T > b.bn || (I % 4) || (split_stride % 4) || (((uintptr_t)gu) & 15) || (((uintptr_t)out) & 7) ||
        (long long)T * I > (1LL << 30))
        return ODIN_ERR_UNSUPPORTED;
    int rc = make_room(0, (cudaStream_t)stream);
    if (rc) return rc;
    SwigluOp s;
    s.gu = gu; s.split_stride = split_stride; s.n_split = n_split; s.out = (bf16*)out; s.T = T; s.I = I;
    ProgOp& op = b.prog.ops[b.prog.n_ops++];
    op.kind = OP_SWIGLU;
    op.s = s;
    return 0;
}

// Decode attention with head preparation; the arguments of odin_attention_decode_fused, with qkv as
// 32-bit partial sums [parts][B][row_stride...].
extern "C" int odin_prog_attention(const float* qkv, int parts, long long part_stride, long long row_stride, void* out,
                                   long long out_row_stride, int B, int Hq, int Hkv, int hd, const void* q_norm_w,
                                   const void* k_norm_w, int w_dtype, int has_norm, float eps, const float* cos_t,
                                   const float* sin_t, int rot, int table_len, void* k_cache, void* v_cache,
                                   int page_size, int n_pages, const int* tok_pos, const int* tok_seq,
                                   const int* block_table, int bt_stride, int window, float* scratch, int n_split,
                                   int write_kv, void* stream) {
    Builder& b = g_builder;
    if (!b.open) return ODIN_ERR_BAD_ARG;
    if (B <= 0 || Hkv <= 0 || Hq % Hkv != 0 || n_split < 1 || scratch == nullptr || parts < 1) return ODIN_ERR_BAD_ARG;
    if (!((hd == 64 || hd == 128) && rot == hd && Hq / Hkv <= 16 && page_size == attn::PAGE_T && n_pages > 0 &&
          (row_stride % 4) == 0 && (part_stride % 4) == 0 && (out_row_stride % 4) == 0 && write_kv &&
          ((((uintptr_t)qkv) | ((uintptr_t)cos_t) | ((uintptr_t)sin_t) | ((uintptr_t)scratch)) & 15) == 0 &&
          (((uintptr_t)out) & 7) == 0))
        return ODIN_ERR_UNSUPPORTED;
    if (B > b.bn || (b.hd != 0 && b.hd != hd) || (long long)B * Hkv > PROG_SPLIT_COUNTERS ||
        (long long)B * Hkv * n_split > (1 << 24))
        return ODIN_ERR_UNSUPPORTED;
    int rc = make_room(2, (cudaStream_t)stream);
    if (rc) return rc;
    for (int j = 0; j < b.prog.n_ops; ++j)
        if (b.prog.ops[j].kind == OP_ATTN) {  // one attention per program: this one starts the next
            if ((rc = run_builder((cudaStream_t)stream))) return rc;
            break;
        }
    const long long rows = (long long)n_pages * Hkv * attn::PAGE_T;
    if ((rc = attn::cache_map(&b.prog.maps[b.n_maps], k_cache, rows, hd))) return rc;
    if ((rc = attn::cache_map(&b.prog.maps[b.n_maps + 1], v_cache, rows, hd))) return rc;
    AttnOp a;
    std::memset(&a, 0, sizeof(a));
    attn_decode::DecodeTcParams& p = b.prog.attn;
    std::memset(&p, 0, sizeof(p));
    p.out = (bf16*)out; p.out_stride = (size_t)out_row_stride;
    p.Hq = Hq; p.Hkv = Hkv; p.tok_pos = tok_pos; p.tok_seq = tok_seq;
    p.block_table = block_table; p.bt_stride = bt_stride; p.window = window;
    p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
    p.part_acc = scratch; p.part_ml = scratch + (size_t)B * Hq * n_split * hd; p.n_split = n_split;
    p.error = device_symbol(g_prog_error, 1);
    p.counters = device_symbol(g_prog_split_counters, 2);
    if (p.counters == nullptr) return ODIN_ERR_UNSUPPORTED;
    p.qkv = qkv; p.qkv_row_stride = (size_t)row_stride; p.qkv_part_stride = (size_t)part_stride; p.qkv_parts = parts;
    p.q_norm = VecRef{q_norm_w, w_dtype == ODIN_BF16}; p.k_norm = VecRef{k_norm_w, w_dtype == ODIN_BF16};
    p.has_norm = has_norm; p.eps = eps; p.cos_t = cos_t; p.sin_t = sin_t; p.table_len = table_len;
    p.k_cache = (bf16*)k_cache; p.v_cache = (bf16*)v_cache; p.write_kv = write_kv;
    a.map = b.n_maps; a.B = B;
    b.n_maps += 2;
    b.hd = hd;
    ProgOp& op = b.prog.ops[b.prog.n_ops++];
    op.kind = OP_ATTN;
    op.a = a;
    return 0;
}

// Reads and clears the flag that a program sets when one of its bounded waits ran out (synchronises the
// device).  0: all well.  out8 (may be null) receives the details of the first wait that ran out.
extern "C" int odin_prog_error(int* out8) {
    int* f = device_symbol(g_prog_error, 1);
    if (f == nullptr) return 0;
    int v[8] = {0};
    if (cudaMemcpy(v, f, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (out8 != nullptr) std::memcpy(out8, v, sizeof(v));
    if (v[0]) {
        cudaMemset(f, 0, sizeof(v));
        // CTAs of the failed launch may never have met: all counters start from zero again
        if (int* c = device_symbol(g_prog_sync, 0)) cudaMemset(c, 0, (2 * MAX_OPS + 1) * sizeof(int));
        if (int* c = device_symbol(g_prog_split_counters, 2)) cudaMemset(c, 0, PROG_SPLIT_COUNTERS * sizeof(int));
    }
    return v[0];
}

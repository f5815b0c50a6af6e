// C[M,N] = A[M,K] * W[N,K]^T for many tokens, on pairs of SMs: tcgen05.mma.cta_group::2.
//
// The one-CTA kernel (gemm_tc.cu) pulls 48 KB from L2 for every 128 x 256 x 64 block of
// products, and that traffic, not the tensor pipe, sets its speed.  Here two CTAs of a
// cluster share one 256 x 256 output tile: each brings its own 128 token rows (A) and its own
// half of the 256 weight rows (B), 32 KB per block and CTA, and the MMA of the pair reads both
// halves of B from the two CTAs' shared memories.  A third less traffic per product, and a
// ring of six stages instead of four.
//
// Roles in each CTA (192 threads): warp 0 issues its TMA loads; warp 1 allocates tensor
// memory, and in the leading CTA (rank 0 of the pair) issues the MMAs for both; warps 2..5
// read the CTA's half of the accumulator back (its 128 rows) and store it.
// Barriers (same offsets in both CTAs):
//   full[s]      in the leader: both CTAs' loads of stage s have landed (the peer's copies
//                complete their bytes on the leader's barrier);
//   empty[s]     in each CTA: the MMAs that read stage s are done (commit to both CTAs);
//   acc_full[a]  in each CTA: accumulator a is complete (commit to both);
//   acc_empty[a] in the leader: both CTAs' epilogues have read accumulator a back.
// DUAL: gate and up products side by side and the SwiGLU in the epilogue, as in gemm_tc.cu.
// WIDE (some hundred tokens): the operands change places: the pair's 256 rows are weight rows, the N
// side holds a tile of 256 tokens (each CTA loads half of it), K is cut into parts, an item is (weight
// tile, K part, tile of tokens), and the epilogue writes C[token][weight row]: a product of so few tokens is bound by the weights it streams, and
// tiles of 256 token rows would be too few to occupy the GPU.
//
// Every wait is bounded (tc::mbar_wait); a CTA that gives up sets the error flag, and both
// CTAs of a pair always reach the final cluster barrier, since no wait of either is endless.
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "tc_common.cuh"

namespace {

constexpr int BM = 128;      // token rows per CTA; the pair's tile has 256
constexpr int BN = 256;      // weight rows of the pair's tile
constexpr int BK = 64;       // K elements per stage: 128 bytes, one swizzle row
constexpr int UMMA_K = 16;
constexpr int ACC_BUFS = 2;
constexpr int STAGE_A = BM * BK * 2;        // 16 KB
constexpr int STAGE_B = (BN / 2) * BK * 2;  // 16 KB: this CTA's half of the weight rows
constexpr int STAGE = STAGE_A + STAGE_B;
constexpr int STAGES = 6;
constexpr int SMEM = STAGES * STAGE + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = ACC_BUFS * BN;    // 512

struct Params2 {
    void* out;
    long long ldc;
    int M, N, K;          // N: output columns (DUAL: the inner size I)
    int tiles_m, tiles_n; // pair tiles: 256 rows x 256 columns (DUAL: 256 x 128)
    int kb_total;
    int dual_offset;      // DUAL: first weight row of the up half
    int accumulate;       // float32 out: C += the product (the residual stream takes its update in place)
    int* error;
    // WIDE (a few hundred tokens): the weights are the operand on the 256-row side (M: weight rows, tiles_m of
    // them, tiles_n = 1) and the tokens the one on the N side (N: tokens, at most 256); K is cut into n_split
    // parts, part s written to the slice s of the output, split_stride elements apart, as C[token][weight row].
    int n_split, kb_per_split;
    long long split_stride;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of the same shared-memory place in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(tc::smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile into this CTA's shared memory; its bytes complete on a barrier given by cluster address
// (the leader's), which the pair form of the copy allows.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(tc::smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(smem_dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem, both CTAs] (+)= A[shared, both] * B[shared, both]^T, issued by one thread of the leader.
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero)
        : "memory");
}
// One arrival on the barrier at this offset in both CTAs when every MMA issued so far is done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(tc::smem_u32(bar)), "h"(mask)
                 : "memory");
}

__device__ __noinline__ void report2(int* err, int what, int tile, int kb, int slot) {
    if (err == nullptr) return;
    if (atomicCAS(err, 0, what) == 0) {
        err[1] = (int)blockIdx.x; err[2] = tile; err[3] = kb; err[4] = slot; err[5] = 2; err[6] = BN; err[7] = (int)gridDim.x;
    }
}

template <typename TO>
__device__ __forceinline__ void store32(TO* dst, const uint32_t* r, int n);
template <>
__device__ __forceinline__ void store32<float>(float* dst, const uint32_t* r, int n) {
    if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    } else {
        for (int i = 0; i < n; ++i) dst[i] = __uint_as_float(r[i]);
    }
}
template <>
__device__ __forceinline__ void store32<bf16>(bf16* dst, const uint32_t* r, int n) {
    if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t p[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]), __uint_as_float(r[8 * i + 2 * j + 1]));
                p[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(p[0], p[1], p[2], p[3]);
        }
    } else {
        for (int i = 0; i < n; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

// Which tile is the w-th?  Tiles are walked in bands of GROUP_M row tiles: within a band the row tile
// runs fastest, then the column tile, so that the clusters at work at one time share a few row tiles'
// tokens and a few column tiles' weights, and a band's tokens stay in L2 while all weights pass by.
// (Row tile fastest over ALL rows, as a first version had it, reads every token once per column tile:
// with 75 k tokens the activations no longer fit L2 and the product ran at the speed of DRAM.)
constexpr int GROUP_M = 8;
__device__ __forceinline__ void tile_of(long long w, int tiles_m, int tiles_n, int& tm, int& tn) {
    const long long band_tiles = (long long)GROUP_M * tiles_n;
    const int band = (int)(w / band_tiles);
    const int in_band = (int)(w - band * band_tiles);
    const int rows = min(GROUP_M, tiles_m - band * GROUP_M);
    tm = band * GROUP_M + in_band % rows;
    tn = in_band / rows;
}

template <typename TO, bool DUAL, bool WIDE = false>
__global__ void __launch_bounds__(192, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params2 p) {
    constexpr int ACC_N = DUAL ? BN / 2 : BN;  // columns of one product of the pair (DUAL: gate and up, 128 each)
    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs: the dynamic shared memory starts at the same place in each
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    uint64_t* full = bars;
    uint64_t* empty = bars + STAGES;
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = acc_full + ACC_BUFS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_BUFS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    pdl_trigger();

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < ACC_BUFS; ++a) {
            tc::mbar_init(&acc_full[a], 1);
            tc::mbar_init(&acc_empty[a], 8);  // four epilogue warps in each of the two CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before either signals the other
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int n_clusters = (int)(gridDim.x >> 1), cluster_id = (int)(blockIdx.x >> 1);
    static_assert(!(DUAL && WIDE), "the SwiGLU epilogue is for many tokens");
    // WIDE: an item is (weight tile, K part, tile of 256 tokens), the tokens' tile running fastest, so that the
    // items that share a weight tile's K part run at about the same time and the second finds it in L2
    const long long n_tiles = WIDE ? (long long)p.tiles_m * p.n_split * p.tiles_n : (long long)p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            pdl_wait();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (long long w = cluster_id; w < n_tiles && ok; w += n_clusters) {
                int tm, tn, kb0 = 0, kb1 = p.kb_total;
                if (WIDE) {
                    const long long rest = w / p.tiles_n;
                    tn = (int)(w % p.tiles_n); tm = (int)(rest / p.n_split);
                    kb0 = (int)(rest % p.n_split) * p.kb_per_split; kb1 = min(p.kb_total, kb0 + p.kb_per_split);
                } else {
                    tile_of(w, p.tiles_m, p.tiles_n, tm, tn);
                }
                const int row_a = tm * 2 * BM + (int)rank * BM;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { report2(p.error, 1, (int)w, kb, stage); ok = false; break; }
                    uint8_t* sa = smem + stage * STAGE;
                    uint8_t* sb = sa + STAGE_A;
                    const uint32_t bar = map_to_rank(&full[stage], 0);
                    if (leader) tc::mbar_expect_tx(&full[stage], 2 * STAGE);  // this CTA's bytes and the peer's
                    tma_load_2d_pair(sa, &map_a, kb * BK, row_a, bar);
                    if (DUAL) {
                        // the pair's gate and up tiles have 128 weight rows each: 64 of each per CTA
                        const int r0 = tn * (BN / 2) + (int)rank * (BN / 4);
                        tma_load_2d_pair(sb, &map_w, kb * BK, r0, bar);
                        tma_load_2d_pair(sb + STAGE_B / 2, &map_w, kb * BK, p.dual_offset + r0, bar);
                    } else {
                        tma_load_2d_pair(sb, &map_w, kb * BK, tn * BN + (int)rank * (BN / 2), bar);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok && leader) {
                // aborted: let the copies already in flight land before the CTA's memory is released
                for (int s2 = 0; s2 < STAGES; ++s2)
                    for (uint32_t i = 0; i < 4096; ++i)
                        if (tc::mbar_try_wait(&full[s2], 0) || tc::mbar_try_wait(&full[s2], 1)) break;
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer (leader only)
        if (leader && lane == 0) {
            // DUAL: a CTA's 64 gate rows and 64 up rows lie one after the other in shared memory, so one
            // MMA over 256 weight rows of the pair gives, in accumulator columns, [gate 0..63 | up 0..63]
            // from the leader's rows and [gate 64..127 | up 64..127] from the peer's
            constexpr uint32_t idesc = tc::make_idesc_bf16(2 * BM, BN);
            uint32_t stage = 0, phase = 0, local = 0;
            bool ok = true;
            pdl_wait();
            for (long long w = cluster_id; w < n_tiles && ok; w += n_clusters, ++local) {
                const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
                if (!tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag)) { report2(p.error, 2, (int)w, -1, (int)acc); ok = false; break; }
                tc::fence_after_sync();
                const uint32_t tmem_d = tmem_base + acc * BN;
                int kb0 = 0, kb1 = p.kb_total;
                if (WIDE) { kb0 = (int)((w / p.tiles_n) % p.n_split) * p.kb_per_split; kb1 = min(p.kb_total, kb0 + p.kb_per_split); }
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!tc::mbar_wait(&full[stage], phase, abort_flag)) { report2(p.error, 3, (int)w, kb, stage); ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t ax = tc::smem_u32(smem + stage * STAGE);
                    const uint64_t da = tc::make_smem_desc_sw128(ax);
                    const uint64_t db = tc::make_smem_desc_sw128(ax + STAGE_A);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit_pair(&acc_full[acc]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int quarter = warp & 3;  // the TMEM lanes this warp may read: [32*quarter, +32)
        pdl_wait();
        uint32_t local = 0;
        bool ok = true;
        const uint32_t acc_empty_leader0 = map_to_rank(&acc_empty[0], 0);
        for (long long w = cluster_id; w < n_tiles && ok; w += n_clusters, ++local) {
            int tm, tn;
            if (WIDE) { tn = (int)(w % p.tiles_n); tm = (int)((w / p.tiles_n) / p.n_split); }
            else tile_of(w, p.tiles_m, p.tiles_n, tm, tn);
            const uint32_t acc = local % ACC_BUFS, acc_phase = (local / ACC_BUFS) & 1;
            if (!tc::mbar_wait(&acc_full[acc], acc_phase, abort_flag)) { if (lane == 0 && quarter == 2) report2(p.error, 4, (int)w, -1, (int)acc); ok = false; break; }
            tc::fence_after_sync();
            const int i = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;  // token row (WIDE: weight row)
            TO* out = reinterpret_cast<TO*>(p.out);
            if (WIDE) {
                // C[token c][weight row i]: the warp writes 32 consecutive elements of a token's row
                const int tok0 = tn * BN;  // first token of this item's tile
                TO* dst = out + (size_t)((w / p.tiles_n) % p.n_split) * p.split_stride + (size_t)tok0 * p.ldc + i;
#pragma unroll 1
                for (int c0 = 0; c0 < BN && tok0 + c0 < p.N; c0 += 32) {
                    uint32_t r[32];
                    tc::tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0, r);
                    tc::tmem_ld_wait();
                    if (i < p.M) {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (tok0 + c0 + c < p.N) dst[(size_t)(c0 + c) * p.ldc] = from_f32<TO>(__uint_as_float(r[c]));
                    }
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < ACC_N; c0 += 32) {
                uint32_t r[32];
                // DUAL: output column c0 + q has its gate in accumulator column c0 + q (+ 64 for the peer's
                // rows, c0 >= 64) and its up 64 columns further
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0 +
                                       ((DUAL && c0 >= BN / 4) ? BN / 4 : 0);
                if (DUAL) {
                    // h = gate * sigmoid(gate) * up (infer/forward.odin:128-133), both halves from TMEM
                    uint32_t u[32];
                    tc::tmem_ld32(taddr, r);
                    tc::tmem_ld32(taddr + BN / 4, u);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 32; ++q) {
                        float g = __uint_as_float(r[q]);
                        g = __fdividef(g, 1.0f + __expf(-g));  // one ex2 and one rcp: the epilogue's arithmetic is not free beside the MMAs
                        r[q] = __float_as_uint(g * __uint_as_float(u[q]));
                    }
                } else {
                    tc::tmem_ld32(taddr, r);
                    tc::tmem_ld_wait();
                }
                const int j0 = tn * ACC_N + c0;
                if (i < p.M && j0 < p.N) {
                    const int n = min(32, p.N - j0);
                    TO* dst = out + (size_t)i * p.ldc + j0;
                    if (std::is_same<TO, float>::value && p.accumulate) {
                        const float* old = reinterpret_cast<const float*>(dst);
                        if (n == 32 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float4 o4 = reinterpret_cast<const float4*>(old)[q];
                                r[4 * q] = __float_as_uint(o4.x + __uint_as_float(r[4 * q]));
                                r[4 * q + 1] = __float_as_uint(o4.y + __uint_as_float(r[4 * q + 1]));
                                r[4 * q + 2] = __float_as_uint(o4.z + __uint_as_float(r[4 * q + 2]));
                                r[4 * q + 3] = __float_as_uint(o4.w + __uint_as_float(r[4 * q + 3]));
                            }
                        } else {
                            for (int q = 0; q < n; ++q) r[q] = __float_as_uint(old[q] + __uint_as_float(r[q]));
                        }
                    }
                    store32<TO>(dst, r, n);
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + acc * 8);
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error != nullptr) atomicCAS(p.error, 0, 99);
    cluster_sync();  // the peer may read this CTA's shared memory and signal its barriers until here
    if (warp == 1) {
        tc::fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn2() {
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

// A row-major [rows, K] bfloat16 matrix with row stride ld, read in boxes of 64 (K) x box_rows,
// 128-byte swizzle, zeros beyond the edges.
int make_map2(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn2();
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

int* error_flag2() {
    static int* flag = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&flag, 8 * sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, 8 * sizeof(int));
        else flag = nullptr;
    });
    return flag;
}

template <typename TO, bool DUAL, bool WIDE = false>
int launch2(const CUtensorMap& ma, const CUtensorMap& mw, const Params2& p, cudaStream_t s) {
    auto kern = gemm_tc2_kernel<TO, DUAL, WIDE>;
    static int max_clusters = -1;
    if (max_clusters < 0) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        cudaLaunchConfig_t q;
        std::memset(&q, 0, sizeof(q));
        q.gridDim = dim3(2 * 74);
        q.blockDim = dim3(192);
        q.dynamicSmemBytes = SMEM;
        cudaLaunchAttribute a[1];
        a[0].id = cudaLaunchAttributeClusterDimension;
        a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
        q.attrs = a;
        q.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &q);
        if (e != cudaSuccess || n <= 0) { cudaGetLastError(); return ODIN_ERR_UNSUPPORTED; }
        max_clusters = n;
    }
    const long long tiles = WIDE ? (long long)p.tiles_m * p.n_split * p.tiles_n : (long long)p.tiles_m * p.tiles_n;
    const int clusters = (int)(tiles < max_clusters ? tiles : max_clusters);
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = odin_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, ma, mw, p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// C[M, N] = A[M, K] W[N, K]^T on pairs of SMs (tiles of 256 x 256); for many tokens.  A: bfloat16, row
// stride lda; W: bfloat16, row stride ldw; C of c_dtype (bfloat16 or float32), row stride ldc.
// Strides and K multiples of 8 elements, pointers 16-byte aligned, else ODIN_ERR_UNSUPPORTED.
// accumulate (float32 C only): C += A W^T, each element read once and written once by the thread that holds its sum.
extern "C" int odin_gemm_tc2(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, long long lda,
                             long long ldw, long long ldc, int accumulate, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    Params2 p;
    p.out = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
    p.tiles_n = (N + BN - 1) / BN;
    p.kb_total = (K + BK - 1) / BK;
    p.dual_offset = 0;
    p.n_split = 1; p.kb_per_split = p.kb_total; p.split_stride = 0;
    if (accumulate && c_dtype != ODIN_F32) return ODIN_ERR_BAD_ARG;
    p.accumulate = accumulate ? 1 : 0;
    p.error = error_flag2();
    CUtensorMap ma, mw;
    int rc;
    if ((rc = make_map2(&ma, A, M, K, lda, BM))) return rc;
    if ((rc = make_map2(&mw, W, N, K, ldw, BN / 2))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (c_dtype == ODIN_BF16) return launch2<bf16, false>(ma, mw, p, s);
    if (c_dtype == ODIN_F32) return launch2<float, false>(ma, mw, p, s);
    return ODIN_ERR_UNSUPPORTED;
}

// C[M, I] = silu(A Wg^T) * (A Wu^T) for W = [Wg; Wu] of shape [2 I, K], on pairs of SMs (tiles of 256 rows
// and 128 output columns: the gate and up products side by side in tensor memory).
extern "C" int odin_gemm_tc2_swiglu(const void* A, const void* W, void* C, int c_dtype, int M, int I, int K,
                                    long long lda, long long ldw, long long ldc, void* stream) {
    if (M <= 0 || I <= 0) return 0;
    if (K <= 0) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    // a box of 64 weight rows must not run from the gate half into the up half
    if (I % (BN / 4) != 0) return ODIN_ERR_UNSUPPORTED;
    Params2 p;
    p.out = C; p.ldc = ldc; p.M = M; p.N = I; p.K = K;
    p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
    p.tiles_n = (I + BN / 2 - 1) / (BN / 2);
    p.kb_total = (K + BK - 1) / BK;
    p.dual_offset = I;
    p.n_split = 1; p.kb_per_split = p.kb_total; p.split_stride = 0;
    p.accumulate = 0;
    p.error = error_flag2();
    CUtensorMap ma, mw;
    int rc;
    if ((rc = make_map2(&ma, A, M, K, lda, BM))) return rc;
    if ((rc = make_map2(&mw, W, 2LL * I, K, ldw, BN / 4))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (c_dtype == ODIN_BF16) return launch2<bf16, true>(ma, mw, p, s);
    if (c_dtype == ODIN_F32) return launch2<float, true>(ma, mw, p, s);
    return ODIN_ERR_UNSUPPORTED;
}

// Some hundred tokens (in tiles of 256): C[n_split][M, N] = A[M, K] W[N, K]^T with the weights on the 256-row side
// of the pair's MMA and the tokens on its N side, each CTA of a pair loading half of the tokens and its 128
// weight rows (32 KB per K block instead of the 48 KB of one CTA with 256 tokens beside it, which bound that
// kernel by its traffic from L2).  K is cut into n_split parts; part s goes to the slice s of C, split_stride
// elements apart (float32 when there is more than one part).
extern "C" int odin_gemm_tc2_wide(const void* A, const void* W, void* C, int c_dtype, int M, int N, int K, long long lda,
                                  long long ldw, long long ldc, int n_split, long long split_stride, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || n_split < 1) return ODIN_ERR_BAD_ARG;
    if ((lda % 8) || (ldw % 8) || (K % 8) || (((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return ODIN_ERR_UNSUPPORTED;
    if (n_split > 1 && c_dtype != ODIN_F32) return ODIN_ERR_BAD_ARG;
    Params2 p;
    p.out = C; p.ldc = ldc; p.M = N; p.N = M; p.K = K;   // the kernel's M side holds the weight rows
    p.tiles_m = (N + 2 * BM - 1) / (2 * BM);
    p.tiles_n = (M + BN - 1) / BN;  // tiles of 256 tokens
    p.kb_total = (K + BK - 1) / BK;
    if (n_split > p.kb_total) n_split = p.kb_total;
    p.kb_per_split = (p.kb_total + n_split - 1) / n_split;
    if ((p.kb_total + p.kb_per_split - 1) / p.kb_per_split != n_split) return ODIN_ERR_BAD_ARG;  // an empty part
    p.n_split = n_split; p.split_stride = split_stride;
    p.dual_offset = 0;
    p.accumulate = 0;
    p.error = error_flag2();
    CUtensorMap ma, mw;
    int rc;
    if ((rc = make_map2(&ma, W, N, K, ldw, BM))) return rc;
    if ((rc = make_map2(&mw, A, M, K, lda, BN / 2))) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (c_dtype == ODIN_BF16) return launch2<bf16, false, true>(ma, mw, p, s);
    if (c_dtype == ODIN_F32) return launch2<float, false, true>(ma, mw, p, s);
    return ODIN_ERR_UNSUPPORTED;
}

// Reads and clears the pair kernel's error flag (synchronises the device).  0: all well; out8: the details
// of the first wait that ran out ([which wait, block, tile, k block, slot, 2, tile width, grid size]).
extern "C" int odin_gemm_tc2_error(int* out8) {
    int* f = error_flag2();
    if (f == nullptr) return 0;
    int v[8] = {0};
    if (cudaMemcpy(v, f, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (out8 != nullptr) std::memcpy(out8, v, sizeof(v));
    if (v[0]) cudaMemset(f, 0, sizeof(v));
    return v[0];
}

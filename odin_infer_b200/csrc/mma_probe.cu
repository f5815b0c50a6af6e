// A measuring tool, not a product kernel: how fast does tcgen05.mma run for the shapes and the
// issue orders that the attention kernels use?  One thread per CTA issues a long run of MMAs on
// constant operands (random bfloat16 of magnitude 1..2 in shared memory; whatever tensor memory
// holds where an operand is read from there) and takes clock64 around the run and the commit that
// ends it.  The results are in cycles of the SM clock, so they do not depend on the clock.
//
// Patterns:
//   0  a run of one shape, A and B from shared memory (M 128, N and B's layout as asked)
//   1  the same with A from tensor memory
//   2  the prompt attention kernel's order for one page of 64 keys and head size 128: four
//      products P V (A from tensor memory, N 128, V MN-major), then the eight score products
//      after next (N 64) into the buffer that P was read from; two score buffers in turn
//   3  two pages a step: eight P V products over 128 keys, then eight score products with N 128
//   4  groups of eight MMAs (A from tensor memory, N 128, B MN-major) each followed by a commit and the wait
//      for it, as a thread issues them that has to wait for its operands in between: the time until the
//      eighth MMA is issued is counted apart (second half of `cycles`), so that one sees whether issuing
//      into an idle tensor core returns at once or takes as long as the MMAs before it run
//   5  the same with A and B from shared memory and N 64
// `commits` adds the commits that a kernel needs after each group of MMAs (to barriers that
// nobody waits on).  Launched with one or two CTAs per SM (the second by a larger or smaller
// shared-memory request), as many CTAs as SMs x that, so that every SM does the same.
// Every wait is bounded.
#include "tc_common.cuh"

namespace {

struct ProbeParams {
    int pattern, n, b_mn, commits, iters, tmem_cols;
    long long* cycles;  // [2 x grid]: the whole run, and for patterns 4 and 5 the part spent issuing
    int* error;
};

constexpr int A_BYTES = 32768, B_BYTES = 65536;

__global__ void __launch_bounds__(128, 2) mma_probe_kernel(const ProbeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + A_BYTES;
    uint64_t* done = reinterpret_cast<uint64_t*>(sB + B_BYTES);
    uint64_t* idle = done + 1;  // [4] barriers that take the commits of the patterns
    uint32_t* slot = reinterpret_cast<uint32_t*>(idle + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(slot + 1);
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        reinterpret_cast<uint32_t*>(smem)[i] = (0x3F80u | (h & 0x807Fu)) | ((0x3F80u | ((h >> 16) & 0x807Fu)) << 16);
    }
    if (threadIdx.x == 0) {
        tc::mbar_init(done, 1);
        for (int i = 0; i < 4; ++i) tc::mbar_init(&idle[i], 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
    }
    tc::fence_proxy_async();
    if (threadIdx.x < 32) tc::tmem_alloc(slot, p.tmem_cols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t t0 = *slot;
    if (threadIdx.x == 0) {
        const uint32_t a_u = tc::smem_u32(sA), b_u = tc::smem_u32(sB);
        const uint32_t a_col = p.tmem_cols - 32;  // where A is read from in tensor memory (pattern 1)
        const long long c0 = clock64();
        if (p.pattern <= 1) {
            const uint32_t idesc = p.b_mn ? tc::make_idesc_bf16_b_mn(128, p.n) : tc::make_idesc_bf16(128, p.n);
            const uint64_t a_d = tc::make_smem_desc_sw128(a_u);
            const uint64_t b_d = p.b_mn ? tc::make_smem_desc_sw128_mn(b_u, 8192, 1024) : tc::make_smem_desc_sw128(b_u);
            const uint64_t b_step = p.b_mn ? (2048 >> 4) : 2;
            for (int i = 0; i < p.iters / 8; ++i) {
                const uint32_t acc = i > 0 ? 1u : 0u;
                if (p.pattern == 0) {
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        tc::umma_bf16(t0, a_d + 2 * (u & 3), b_d + b_step * (u & 3), idesc, u > 0 ? 1u : acc);
                } else {
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        tc::umma_bf16_ts(t0, t0 + a_col + 8 * (u & 3), b_d + b_step * (u & 3), idesc, u > 0 ? 1u : acc);
                }
            }
        } else if (p.pattern == 2) {
            constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 64);
            constexpr uint32_t idesc_o = tc::make_idesc_bf16_b_mn(128, 128);
            for (int i = 0; i < p.iters; ++i) {
                const int st = i & 1;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    tc::umma_bf16_ts(t0 + 128, t0 + st * 64 + j * 8,
                                     tc::make_smem_desc_sw128_mn(b_u + 16384 + j * 2048, 8192, 1024), idesc_o,
                                     (i > 0 || j > 0) ? 1u : 0u);
                if (p.commits >= 1) tc::umma_commit(&idle[0]);
                if (p.commits >= 2) tc::umma_commit(&idle[1]);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc::umma_bf16(t0 + st * 64, tc::make_smem_desc_sw128(a_u + (k >> 2) * 16384 + (k & 3) * 32),
                                  tc::make_smem_desc_sw128(b_u + (k >> 2) * 8192 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                if (p.commits >= 1) tc::umma_commit(&idle[2]);
                if (p.commits >= 2) tc::umma_commit(&idle[3]);
            }
        } else if (p.pattern >= 4) {
            constexpr uint32_t idesc_o = tc::make_idesc_bf16_b_mn(128, 128);
            constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 64);
            long long issue = 0;
            bool ok = true;
            for (int i = 0; i < p.iters && ok; ++i) {
                const long long g0 = clock64();
                if (p.pattern == 4) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        tc::umma_bf16_ts(t0 + 128, t0 + j * 8, tc::make_smem_desc_sw128_mn(b_u + 32768 + j * 2048, 16384, 1024),
                                         idesc_o, (i > 0 || j > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        tc::umma_bf16(t0, tc::make_smem_desc_sw128(a_u + (k >> 2) * 16384 + (k & 3) * 32),
                                      tc::make_smem_desc_sw128(b_u + (k >> 2) * 8192 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                }
                issue += clock64() - g0;
                tc::umma_commit(&idle[0]);
                ok = tc::mbar_wait(&idle[0], i & 1, abort_flag);
                tc::fence_after_sync();
            }
            p.cycles[gridDim.x + blockIdx.x] = issue;
        } else {
            constexpr uint32_t idesc_s = tc::make_idesc_bf16(128, 128);
            constexpr uint32_t idesc_o = tc::make_idesc_bf16_b_mn(128, 128);
            for (int i = 0; i < p.iters; ++i) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    tc::umma_bf16_ts(t0 + 128, t0 + j * 8, tc::make_smem_desc_sw128_mn(b_u + 32768 + j * 2048, 16384, 1024),
                                     idesc_o, (i > 0 || j > 0) ? 1u : 0u);
                if (p.commits >= 1) tc::umma_commit(&idle[0]);
                if (p.commits >= 2) tc::umma_commit(&idle[1]);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc::umma_bf16(t0, tc::make_smem_desc_sw128(a_u + (k >> 2) * 16384 + (k & 3) * 32),
                                  tc::make_smem_desc_sw128(b_u + (k >> 2) * 16384 + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
                if (p.commits >= 1) tc::umma_commit(&idle[2]);
                if (p.commits >= 2) tc::umma_commit(&idle[3]);
            }
        }
        tc::umma_commit(done);
        const bool ok = tc::mbar_wait(done, 0, abort_flag);
        p.cycles[blockIdx.x] = clock64() - c0;
        if (!ok && p.error != nullptr) atomicExch(p.error, 1);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc::fence_after_sync();
        tc::tmem_dealloc(t0, p.tmem_cols);
    }
}

int* probe_error_flag() {
    static int* flag = nullptr;
    if (flag == nullptr && cudaMalloc(&flag, sizeof(int)) == cudaSuccess) cudaMemset(flag, 0, sizeof(int));
    return flag;
}

}  // namespace

// cycles: [2 * SMs * per_sm] 64-bit counts on the device: one per CTA, then (patterns 4 and 5) one per CTA for the issuing.  iters: MMAs of the run
// (patterns 0 and 1, a multiple of 8), pages / page pairs (patterns 2 and 3) or groups (4 and 5).
extern "C" int odin_mma_probe(int pattern, int n, int b_mn, int commits, int per_sm, int iters, void* cycles,
                              void* stream) {
    if (pattern < 0 || pattern > 5 || per_sm < 1 || per_sm > 2 || iters < 8 || iters > 65536) return ODIN_ERR_BAD_ARG;
    if (pattern <= 1 && (n < 16 || n > 256 || n % 16 != 0 || iters % 8 != 0)) return ODIN_ERR_BAD_ARG;
    if (pattern <= 1 && b_mn && n % 64 != 0) return ODIN_ERR_BAD_ARG;
    if (pattern == 1 && per_sm == 2 && n > 224) return ODIN_ERR_BAD_ARG;  // the accumulator and A share 256 columns
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    ProbeParams p;
    p.pattern = pattern; p.n = n; p.b_mn = b_mn; p.commits = commits; p.iters = iters;
    p.tmem_cols = per_sm == 2 ? 256 : 512;
    p.cycles = (long long*)cycles;
    p.error = probe_error_flag();
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) return ODIN_ERR_UNSUPPORTED;
    const int grid = sms * per_sm;
    // two CTAs fit an SM with 112 KB each and one with 200 KB
    mma_probe_kernel<<<grid, 128, per_sm == 2 ? 112 * 1024 : 200 * 1024, (cudaStream_t)stream>>>(p);
    ODIN_LAUNCH_CHECK();
    return 0;
}

// Reads and clears the flag that the kernel sets when its wait ran out (synchronises the device).
extern "C" int odin_mma_probe_error() {
    int* f = probe_error_flag();
    if (f == nullptr) return 0;
    int v = 0;
    if (cudaMemcpy(&v, f, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(f, 0, sizeof(int));
    return v;
}

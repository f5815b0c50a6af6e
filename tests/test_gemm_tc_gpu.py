"""The tcgen05 matrix product alone against a float64 reference: structured inputs
first (all ones gives K, an identity copies, rows and columns that differ), then
random ones; both operand modes, every tile width, ragged edges, K tails, split-K."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, ref, rtol, what=""):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= rtol, f"{what}: relative error {err:.3e} > {rtol:.1e}"


def run(a, w, mode, bn, out_dtype, n_split=1):
    from odin_infer_b200.csrc import ops
    M, N = a.shape[0], w.shape[0]
    if n_split > 1:
        s = ops.gemm_tc_splits(a.shape[1], n_split)
        out = torch.full((s, M, N), float("nan"), device=DEV, dtype=torch.float32)
        ops.gemm_tc(a, w, out, mode, bn, n_split)
        ops.gemm_tc_check()
        assert not torch.isnan(out).any()
        return out.sum(0)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    ops.gemm_tc(a, w, out, mode, bn)
    ops.gemm_tc_check()
    assert not torch.isnan(out.float()).any()
    return out


CASES = [
    # (M, N, K, mode, bn)
    (128, 256, 64, 0, 256), (128, 128, 128, 0, 128), (2048, 512, 256, 0, 256), (300, 200, 96, 0, 64),
    (129, 1000, 72, 0, 256), (130, 40, 1032, 0, 64), (1000, 384, 4096, 0, 128),
    (1, 128, 64, 1, 16), (1, 384, 96, 1, 16), (8, 6144, 4096, 1, 16), (16, 300, 72, 1, 16), (17, 256, 128, 1, 32),
    (64, 1000, 1032, 1, 64), (100, 512, 256, 1, 128), (33, 12288, 512, 1, 64),
    (256, 512, 256, 1, 256), (129, 1000, 1032, 1, 256), (200, 300, 72, 1, 256),   # a few hundred tokens, weights wide
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_ladder(case, out_dtype):
    M, N, K, mode, bn = case
    ladder(lambda a, w: run(a, w, mode, bn, out_dtype), M, N, K, out_dtype)


def ladder(run_product, M, N, K, out_dtype):
    """Structured inputs first, random ones last (gemm_harness/gemm_test.odin:1063-1072)."""
    def run(a, w, *_):
        return run_product(a, w)
    mode = bn = None
    exact = 1e-6 if out_dtype == torch.float32 else 4e-3
    ones_a = torch.ones(M, K, device=DEV, dtype=torch.bfloat16)
    ones_w = torch.ones(N, K, device=DEV, dtype=torch.bfloat16)
    close(run(ones_a, ones_w, mode, bn, out_dtype), torch.full((M, N), float(K)), exact, "ones")
    eye = torch.eye(N, K, device=DEV, dtype=torch.bfloat16)
    a = torch.randn(M, K, device=DEV).bfloat16()
    close(run(a, eye, mode, bn, out_dtype), a.double() @ eye.double().t(), exact, "identity")
    rows = (torch.arange(M, device=DEV)[:, None].expand(M, K) % 7).bfloat16().contiguous()
    cols = ((torch.arange(N, device=DEV)[:, None].expand(N, K) % 5) * 0.25).bfloat16().contiguous()
    close(run(rows, cols, mode, bn, out_dtype), rows.double() @ cols.double().t(), exact, "rows/columns")
    # every (row, k) and (column, k) distinct: a wrong swizzle or K step shows as a wrong sum
    ka = ((torch.arange(M, device=DEV)[:, None] * 3 + torch.arange(K, device=DEV)[None, :] * 5) % 11 - 5).bfloat16()
    kw = ((torch.arange(N, device=DEV)[:, None] * 7 + torch.arange(K, device=DEV)[None, :] * 2) % 13 - 6).bfloat16()
    close(run(ka, kw, mode, bn, out_dtype), ka.double() @ kw.double().t(), exact, "k-distinct")
    w = torch.randn(N, K, device=DEV).bfloat16()
    close(run(a, w, mode, bn, out_dtype), a.double() @ w.double().t(),
          (2e-7 * math.sqrt(K) if out_dtype == torch.float32 else 5e-3), "random")


@pytest.mark.parametrize("case", [(8, 4096, 12288, 1, 16, 6), (64, 512, 1032, 1, 64, 4), (3, 256, 640, 1, 16, 4),
                                  (200, 300, 4096, 0, 128, 3), (5, 128, 96, 1, 16, 7), (250, 1000, 4096, 1, 256, 5)])
def test_split_k(case):
    M, N, K, mode, bn, n_split = case
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    close(run(a, w, mode, bn, torch.float32, n_split), a.double() @ w.double().t(), 2e-7 * math.sqrt(K), "split")


@pytest.mark.parametrize("case", [
    # (M, N, K, bn, n_split, stages, staged)
    (8, 6144, 4096, 16, 3, 5, 15),      # q|k|v of the 8B shape beside attention: 20 of a CTA's 22 blocks before the wait
    (8, 4096, 4096, 16, 4, 5, 15),      # o: all 16 blocks of an item staged or in the ring
    (8, 24576, 4096, 16, 3, 0, 15),     # gate|up: four items a CTA, the first one staged
    (3, 384, 1032, 16, 1, 0, 15),       # a K tail, fewer items than CTAs, more blocks staged than the ring is long
    (16, 1000, 4096, 16, 2, 3, 15),     # a ring of three: the staged blocks pass through it five times
    (30, 2048, 2048, 32, 2, 4, 12),     # 32 tokens
    (5, 128, 64, 16, 1, 0, 15),         # one K block
    (8, 1024, 8192, 16, 1, 0, 40),      # more asked for than tensor memory holds
])
def test_weights_staged_in_tensor_memory(case):
    """The first K blocks of a CTA's first item wait in tensor memory (tcgen05.cp from the ring, then MMAs with A
    from tensor memory): the same bits as without, on the ladder's structured inputs and on random ones."""
    from odin_infer_b200.csrc import ops
    M, N, K, bn, n_split, stages, staged = case

    def product(a, w, staged_blocks):
        ns = ops.gemm_tc_splits(K, n_split)
        out = torch.full((ns, M, N), float("nan"), device=DEV, dtype=torch.float32)
        ops.gemm_tc(a, w, out, 1, bn, n_split, stages, staged_blocks)
        ops.gemm_tc_check()
        assert not torch.isnan(out).any()
        return out

    ladder(lambda a, w: product(a, w, staged).sum(0), M, N, K, torch.float32)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    plain = product(a, w, 0)
    for _ in range(3):
        assert torch.equal(product(a, w, staged), plain)


def test_tensor_memory_staging_copy():
    """tcgen05.cp of a swizzled 128 x 64 tile: row m lands in lane m, elements 2c and 2c + 1 in column c."""
    import ctypes
    from odin_infer_b200.csrc import build, ops
    f = build.load("gemm_tc").odin_gemm_tc_stage_probe
    f.restype = ctypes.c_int
    x = torch.randn(128, 64, device=DEV).bfloat16().contiguous()
    out = torch.full((128, 32), -1, dtype=torch.int32, device=DEV)
    assert f(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()),
             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    ops.gemm_tc_check()
    assert torch.equal(out.view(torch.bfloat16).view(128, 64), x)


def test_strided_views_and_batch_invariance():
    """A row's result must not depend on the other rows (same mode, tile and split)."""
    from odin_infer_b200.csrc import ops
    K, N = 1024, 640
    big = torch.randn(40, 2 * K, device=DEV).bfloat16()
    a = big[:, :K]                       # row stride 2K
    w = torch.randn(N, K, device=DEV).bfloat16()
    full = run(a, w, 1, 64, torch.float32)
    close(full, a.double() @ w.double().t(), 2e-7 * math.sqrt(K))
    one = run(a[7:8], w, 1, 64, torch.float32)
    assert torch.equal(one[0], full[7])
    few = run(a[5:17], w, 1, 64, torch.float32)
    assert torch.equal(few, full[5:17])
    sp_full = run(a, w, 1, 64, torch.float32, 4)
    sp_one = run(a[7:8], w, 1, 64, torch.float32, 4)
    assert torch.equal(sp_one[0], sp_full[7])


def test_refuses_what_it_cannot_do():
    from odin_infer_b200.csrc import ops
    a = torch.randn(4, 100, device=DEV).bfloat16()   # K not a multiple of 8
    w = torch.randn(16, 100, device=DEV).bfloat16()
    assert not ops.gemm_tc_supported(a, w)
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(a, w, torch.empty(4, 16, device=DEV, dtype=torch.bfloat16), 1, 16)


@pytest.mark.parametrize("shape", [(129, 128, 64), (300, 200, 96), (2048, 1024, 512), (500, 333 * 8, 72)])
def test_fused_swiglu_product(shape):
    """The gate and up products with the SwiGLU in the epilogue against the two-step computation."""
    from odin_infer_b200.csrc import ops
    M, I, K = shape
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) / math.sqrt(K)).bfloat16()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc_swiglu(a, w, out)
    ops.gemm_tc_check()
    g = a.double() @ w[:I].double().t()
    u = a.double() @ w[I:].double().t()
    close(out, g * torch.sigmoid(g) * u, 6e-3, "fused swiglu")
    # structured: gate rows all equal, up rows count the column: out = silu(c) * j-dependent value
    w2 = torch.zeros(2 * I, K, device=DEV)
    w2[:I, 0] = 1.0
    w2[I:, 1] = torch.arange(I, device=DEV, dtype=torch.float32) % 13
    a2 = torch.zeros(M, K, device=DEV)
    a2[:, 0] = 2.0
    a2[:, 1] = (torch.arange(M, device=DEV) % 5).float()
    ops.gemm_tc_swiglu(a2.bfloat16(), w2.bfloat16(), out)
    ref = (2.0 * torch.sigmoid(torch.tensor(2.0))).item() * (a2[:, 1:2].double() * w2[I:, 1].double()[None, :])
    close(out, ref, 5e-3, "fused swiglu structured")


@pytest.mark.parametrize("stages", [2, 3, 6])
@pytest.mark.parametrize("case", [(8, 6144, 4096, 1, 16, 3), (64, 1000, 1032, 1, 64, 1), (300, 512, 1024, 0, 256, 1)])
def test_short_ring_gives_the_same_result(case, stages):
    """A ring of fewer stages (room for a neighbour on the SM) changes no bit of the result."""
    from odin_infer_b200.csrc import ops
    M, N, K, mode, bn, n_split = case
    torch.manual_seed(stages)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    shape = (ops.gemm_tc_splits(K, n_split), M, N) if n_split > 1 else (M, N)
    full = torch.empty(shape, device=DEV, dtype=torch.float32)
    short = torch.full(shape, float("nan"), device=DEV, dtype=torch.float32)
    ops.gemm_tc(a, w, full, mode, bn, n_split)
    ops.gemm_tc(a, w, short, mode, bn, n_split, stages)
    ops.gemm_tc_check()
    assert torch.equal(full, short)


PAIR_CASES = [(256, 256, 64), (256, 512, 128), (300, 1000, 1032), (129, 200, 72), (2048, 768, 4096), (1000, 6144, 512),
              (513, 264, 96)]


@pytest.mark.parametrize("case", PAIR_CASES)
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_pair_kernel_ladder(case, out_dtype):
    """The two-CTA kernel (tiles of 256 x 256 on pairs of SMs): structured inputs, then random ones; ragged
    edges in M, N and K; more tiles than clusters; each result also against the one-CTA kernel."""
    from odin_infer_b200.csrc import ops
    M, N, K = case
    exact = 1e-6 if out_dtype == torch.float32 else 4e-3

    def run2(a, w):
        out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
        ops.gemm_tc2(a, w, out)
        ops.gemm_tc_check()
        assert not torch.isnan(out.float()).any()
        return out

    ones_a = torch.ones(M, K, device=DEV, dtype=torch.bfloat16)
    ones_w = torch.ones(N, K, device=DEV, dtype=torch.bfloat16)
    close(run2(ones_a, ones_w), torch.full((M, N), float(K)), exact, "ones")
    rows = (torch.arange(M, device=DEV)[:, None].expand(M, K) % 7).bfloat16().contiguous()
    cols = ((torch.arange(N, device=DEV)[:, None].expand(N, K) % 5) * 0.25).bfloat16().contiguous()
    close(run2(rows, cols), rows.double() @ cols.double().t(), exact, "rows x columns")
    eye = torch.eye(N, K, device=DEV, dtype=torch.bfloat16)
    a = torch.randn(M, K, device=DEV).bfloat16()
    close(run2(a, eye), a.double() @ eye.double().t(), exact, "identity")
    torch.manual_seed(M + N + K)
    w = torch.randn(N, K, device=DEV).bfloat16()
    got = run2(a, w)
    tol = 1e-7 * math.sqrt(K) * 8 if out_dtype == torch.float32 else 4e-3
    close(got, a.double() @ w.double().t(), tol, "random")
    one = torch.empty(M, N, device=DEV, dtype=out_dtype)
    ops.gemm_tc(a, w, one, 0, 256)
    close(got, one, 1e-6 if out_dtype == torch.float32 else 8e-3, "against the one-CTA kernel")


@pytest.mark.parametrize("case", [(256, 512, 256, 1), (129, 1000, 1032, 3), (200, 300, 72, 1), (250, 4096, 4096, 5),
                                  (192, 6144, 4096, 3), (1, 256, 64, 1), (130, 40, 640, 10),
                                  (257, 512, 256, 2), (512, 4096, 1024, 4), (700, 300, 1032, 3)])   # several tiles of tokens
def test_pair_kernel_weights_wide(case):
    """The two-CTA kernel for a few hundred tokens (weights on the 256-row side, tokens on the N side, K in
    parts): structured inputs, then random ones; ragged edges in tokens, weight rows and K; a row's result does
    not depend on the other rows."""
    from odin_infer_b200.csrc import ops
    M, N, K, n_split = case
    parts = ops.gemm_tc_splits(K, n_split)

    def run_wide(a, w, dtype=torch.float32):
        m = a.shape[0]
        out = torch.full((parts, m, N) if parts > 1 else (m, N), float("nan"), device=DEV, dtype=dtype)
        ops.gemm_tc2_wide(a, w, out, n_split)
        ops.gemm_tc_check()
        assert not torch.isnan(out.float()).any()
        return out.sum(0) if parts > 1 else out

    ones_a = torch.ones(M, K, device=DEV, dtype=torch.bfloat16)
    ones_w = torch.ones(N, K, device=DEV, dtype=torch.bfloat16)
    close(run_wide(ones_a, ones_w), torch.full((M, N), float(K)), 1e-6, "ones")
    ka = ((torch.arange(M, device=DEV)[:, None] * 3 + torch.arange(K, device=DEV)[None, :] * 5) % 11 - 5).bfloat16()
    kw = ((torch.arange(N, device=DEV)[:, None] * 7 + torch.arange(K, device=DEV)[None, :] * 2) % 13 - 6).bfloat16()
    close(run_wide(ka, kw), ka.double() @ kw.double().t(), 1e-6, "k-distinct")
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = torch.randn(N, K, device=DEV).bfloat16()
    got = run_wide(a, w)
    close(got, a.double() @ w.double().t(), 2e-7 * math.sqrt(K), "random")
    if parts == 1:
        close(run_wide(a, w, torch.bfloat16), a.double() @ w.double().t(), 5e-3, "random, bfloat16 out")
    r = M // 2
    assert torch.equal(run_wide(a[r:r + 1], w)[0], got[r])


@pytest.mark.parametrize("case", [(256, 128, 64), (300, 192, 1032), (2048, 1536, 512), (130, 64, 128)])
def test_pair_kernel_swiglu(case):
    """The two-CTA kernel with the SwiGLU in its epilogue against the formula in float64."""
    from odin_infer_b200.csrc import ops
    M, I, K = case
    torch.manual_seed(I + K)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(2 * I, K, device=DEV) / math.sqrt(K)).bfloat16()
    out = torch.full((M, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.gemm_tc2_swiglu(a, w, out)
    ops.gemm_tc_check()
    g = a.double() @ w[:I].double().t()
    u = a.double() @ w[I:].double().t()
    close(out, g * torch.sigmoid(g) * u, 8e-3, "swiglu")


@pytest.mark.parametrize("case", [(256, 256, 64), (300, 1000, 1032), (2048, 4096, 512)])
def test_pair_kernel_adds_in_place(case):
    """C += A W^T in the epilogue: exactly the separate product added to C."""
    from odin_infer_b200.csrc import ops
    M, N, K = case
    torch.manual_seed(K)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    x0 = torch.randn(M, N, device=DEV)
    prod = torch.empty(M, N, device=DEV)
    ops.gemm_tc2(a, w, prod)
    x = x0.clone()
    ops.gemm_tc2(a, w, x, accumulate=True)
    ops.gemm_tc_check()
    assert torch.equal(x, x0 + prod)


# A product with the fault that the reference keeps beside its kernels to prove that its ladder can fail
# (gemm_harness/gemm_test.odin:322-338, "K-step-16 reproduces the old 2048 bug"): the loop over K advances
# by two blocks and multiplies one.  Compiled here, from this string, at test time; it is in no library.
KNOWN_BAD = r"""
#include <cuda_bf16.h>
__global__ void bad_product(const __nv_bfloat16* A, const __nv_bfloat16* W, float* C, int M, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
    if (n >= N || m >= M) return;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 16)                       // the fault: 16 instead of 8
        for (int k = k0; k < k0 + 8 && k < K; ++k)
            acc = fmaf(__bfloat162float(A[(size_t)m * K + k]), __bfloat162float(W[(size_t)n * K + k]), acc);
    C[(size_t)m * N + n] = acc;
}
extern "C" int bad_product_launch(const void* A, const void* W, float* C, int M, int N, int K, void* stream) {
    bad_product<<<dim3((N + 127) / 128, M), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W, C, M, N, K);
    return (int)cudaGetLastError();
}
"""


def test_ladder_catches_a_known_bad_product(tmp_path):
    """The regression guard of the ladder itself: a product that skips every second block of K must
    fail at the first rung (all ones gives K/2), and with the names of the later rungs too."""
    import ctypes
    import subprocess
    from odin_infer_b200.csrc import build
    src, lib = tmp_path / "bad.cu", tmp_path / "libbad.so"
    src.write_text(KNOWN_BAD)
    nvcc = build._nvcc()
    assert nvcc is not None, "nvcc is needed to build the known-bad variant"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-Xcompiler", "-fPIC", "-shared",
                    "-o", str(lib), str(src)], check=True, capture_output=True)
    fn = ctypes.CDLL(str(lib)).bad_product_launch

    def bad(a, w):
        out = torch.empty(a.shape[0], w.shape[0], device=DEV)
        rc = fn(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                a.shape[0], w.shape[0], a.shape[1], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        return out
    ones = torch.ones(8, 4096, device=DEV, dtype=torch.bfloat16)
    assert bad(ones, ones)[0, 0].item() == 2048.0             # the reference's "old 2048 bug"
    with pytest.raises(AssertionError, match="ones"):
        ladder(bad, 64, 64, 4096, torch.float32)
    with pytest.raises(AssertionError, match="ones"):
        ladder(bad, 8, 8, 16, torch.float32)
    ladder(bad, 8, 8, 8, torch.float32)                       # one block of K: nothing is skipped yet, as in the reference's first rung

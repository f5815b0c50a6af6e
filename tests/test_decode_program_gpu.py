"""The decode step as programs of one persistent kernel (csrc/decode_program.cu, off by default):
the same operations as kernels of their own give the same numbers, through the `ops` wrappers
that record them and through the engine."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def chain(ops, x, delta, w_norm, w_up, w_down, inner, parts):
    """norm(x + delta) -> gate/up product -> SwiGLU -> down product -> norm, as a layer's second half
    does; returns everything that was written."""
    M, d = x.shape
    h = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(x, delta, w_norm, 1e-5, h)
    n1 = ops.gemm_tc_splits(d, parts)
    gu = torch.empty(n1, M, 2 * inner, device=DEV, dtype=torch.float32)
    ops.gemm_tc(h, w_up, gu, 1, 16 if M <= 16 else 32 if M <= 32 else 64, n1)
    act = torch.empty(M, inner, device=DEV, dtype=torch.bfloat16)
    ops.swiglu(gu, act)
    n2 = ops.gemm_tc_splits(inner, parts)
    down = torch.empty(n2, M, d, device=DEV, dtype=torch.float32)
    ops.gemm_tc(act, w_down, down, 1, 16 if M <= 16 else 32 if M <= 32 else 64, n2)
    h2 = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(x, down, w_norm, 1e-5, h2)
    return h, gu, act, down, h2, x


@pytest.mark.parametrize("case", [(8, 512, 1024, 3), (1, 72, 200, 1), (33, 1032, 520, 4), (64, 4096, 1536, 5)])
def test_program_equals_the_kernels_of_their_own(case):
    from odin_infer_b200.csrc import ops
    M, d, inner, parts = case
    torch.manual_seed(d)
    x0 = torch.randn(M, d, device=DEV)
    delta = torch.randn(3, M, d, device=DEV) * 0.3
    w_norm = (1.0 + 0.1 * torch.randn(d, device=DEV)).to(torch.bfloat16)
    w_up = (torch.randn(2 * inner, d, device=DEV) / math.sqrt(d)).to(torch.bfloat16)
    w_down = (torch.randn(d, inner, device=DEV) / math.sqrt(inner)).to(torch.bfloat16)
    ref = chain(ops, x0.clone(), delta, w_norm, w_up, w_down, inner, parts)
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    with ops.program(ops.program_bucket(M)):
        got = chain(ops, x0.clone(), delta, w_norm, w_up, w_down, inner, parts)
    torch.cuda.synchronize()
    ops.program_check()
    ops.gemm_tc_check()
    assert ops.launch_count() - n0 == 1, "six operations, one launch"
    for name, a, b in zip(("normed", "gate/up sums", "activation", "down sums", "normed again", "residual"), got, ref):
        a, b = a.double(), b.double()
        err = (a - b).abs().max().item() / max(b.abs().max().item(), 1e-30)
        # The products and the SwiGLU add in the same order as the kernels of their own; the norm adds up
        # its sum of squares in another order, so a normed element may land on the neighbouring
        # bfloat16 (2^-8 of its size), and what follows moves by as much.
        assert err <= 8e-3, (name, err)


def test_other_kernels_between_operations_keep_their_place():
    """A kernel that a program cannot hold runs after the operations recorded before it."""
    from odin_infer_b200.csrc import ops
    M, d = 4, 256
    torch.manual_seed(1)
    x = torch.randn(M, d, device=DEV)
    w = torch.ones(d, device=DEV, dtype=torch.bfloat16)
    h = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    as32 = torch.empty(M, d, device=DEV, dtype=torch.float32)
    with ops.program(16):
        ops.add_rmsnorm(x, None, w, 1e-6, h)   # recorded
        ops.cast(h, as32)                      # not part of a program: flushes, then runs
    torch.cuda.synchronize()
    ops.program_check()
    ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6)
    assert (as32.double() - ref).abs().max().item() <= 2e-2
    assert not ops.recording()


@pytest.mark.parametrize("graphs", [False, True])
def test_engine_steps_as_programs(graphs, tmp_path, monkeypatch):
    """Decoding through the engine, eagerly and as replayed graphs: the logits of the program path
    against those of the kernel-per-operation path (tiny E: head size 128, so attention is an
    operation of the program too)."""
    import numpy as np
    from tests import tiny
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine import runtime
    raw, seed = tiny.TINIES["E"]
    folder = tiny.make_folder(tmp_path, raw, seed)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, raw["vocab_size"], n).tolist() for n in (70, 3, 129, 64)]
    feed = rng.integers(0, raw["vocab_size"], (40, len(prompts)))
    out = {}
    for program in (False, True):
        monkeypatch.setattr(runtime, "DECODE_PROGRAM", program)
        engine = Engine.load(folder, Engine_Opts(max_ctx=256, max_tokens=4 * 256, dtype="bfloat16", verbose=False,
                                                 cuda_graphs=graphs))
        try:
            slots = [engine.take_slot() for _ in prompts]
            engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
            n0 = ops.launch_count()
            rows = [engine.step([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, toks)]).float().cpu() for toks in feed]
            torch.cuda.synchronize()
            ops.program_check()
            out[program] = (torch.stack(rows), ops.launch_count() - n0)
        finally:
            engine.destroy()
    a, b = out[True][0].double(), out[False][0].double()
    assert (a - b).abs().max().item() <= 2e-2 * b.abs().max().item()
    assert out[True][1] < out[False][1], "a layer's operations share launches"

"""The entry point that allocates nothing, called through its exported C symbol.

Who needs it: a caller that must not (or cannot) allocate device memory when it runs
attention, e.g. a host program that gave all device memory to an arena of its own, or
a loop in which cudaMalloc's device-wide synchronisation is not acceptable.  The
ordinary entry point wants scratch memory from its caller; this one uses a fixed array
inside the library.  The test calls it twice in a row, on different inputs, and
compares each result with the ordinary entry point's, within the tolerance that the
kernel tests use; it also checks that a request beyond the array's size is refused.

This file sorts after the other tests on purpose: a run that stops at the first
failure has then already run everything else.
"""
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def build_case(seed, n_q, n_kv, hd, lengths):
    torch.manual_seed(seed)
    B = len(lengths)
    pages_per = [(n + PAGE - 1) // PAGE for n in lengths]
    total = sum(pages_per) + 2
    order = torch.randperm(total).tolist()
    bt = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    it = iter(order)
    for s, n in enumerate(pages_per):
        for p in range(n):
            bt[s, p] = next(it)
    k = torch.randn(total, n_kv, PAGE, hd, device=DEV).bfloat16()
    v = torch.randn(total, n_kv, PAGE, hd, device=DEV).bfloat16()
    q = torch.randn(B, n_q * hd, device=DEV).bfloat16()
    tok_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    tok_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    return q, k, v, tok_pos, tok_seq, bt.to(DEV)


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    from odin_infer_b200.csrc import build, ops
    lib = build.load("attention_decode")
    fn = lib.odin_attention_decode_noalloc
    fn.restype = c_int
    need = lib.odin_attention_decode_noalloc_need
    need.restype = c_longlong
    n_q, n_kv, hd = 8, 2, 128
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (seed, lengths, n_split) in enumerate([(1, [200, 1, 65, 333], 4), (2, [64, 500, 7], 3)]):
        q, k, v, tok_pos, tok_seq, bt = build_case(seed, n_q, n_kv, hd, lengths)
        B = len(lengths)
        ref = torch.empty(B, n_q * hd, device=DEV, dtype=torch.bfloat16)
        scratch = torch.empty(ops.attention_decode_scratch(B, n_q, hd, n_split), device=DEV)
        ops.attention_decode(q, ref, n_q, n_kv, hd, k, v, tok_pos, tok_seq, bt, 0, scratch, n_split)
        out = torch.zeros_like(ref)
        torch.cuda.synchronize()
        # the device's own count of free memory, which sees every allocation of the process (a
        # cudaMalloc inside the library too), not just those of torch's allocator
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(c_void_p(q.data_ptr()), c_longlong(q.stride(0)), c_void_p(out.data_ptr()), c_longlong(out.stride(0)),
                c_int(B), c_int(n_q), c_int(n_kv), c_int(hd), c_void_p(k.data_ptr()), c_void_p(v.data_ptr()),
                c_int(PAGE), c_int(k.shape[0]), c_void_p(tok_pos.data_ptr()), c_void_p(tok_seq.data_ptr()), c_void_p(bt.data_ptr()),
                c_int(bt.stride(0)), c_int(0), c_int(n_split), stream)
        assert rc == 0, f"call {call}: error code {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call took device memory"
        assert need(c_int(B), c_int(n_q), c_int(hd), c_int(n_split)) == B * n_q * n_split * (hd + 2)
        err = (out.double() - ref.double()).abs().max().item() / ref.double().abs().max().item()
        assert err <= 1e-2, f"call {call}: relative error {err:.3e}"
    # beyond the array's size: refused, nothing launched, the output untouched
    B_big = 4096
    assert need(c_int(B_big), c_int(64), c_int(128), c_int(16)) > (1 << 20)
    marker = torch.full((4,), 3.0, device=DEV)
    rc = fn(c_void_p(marker.data_ptr()), c_longlong(0), c_void_p(marker.data_ptr()), c_longlong(0), c_int(B_big),
            c_int(64), c_int(8), c_int(128), c_void_p(0), c_void_p(0), c_int(PAGE), c_int(0), c_void_p(0), c_void_p(0),
            c_void_p(0), c_int(0), c_int(0), c_int(16), stream)
    assert rc == -4
    torch.cuda.synchronize()
    assert marker.tolist() == [3.0] * 4

"""Times one kernel of this package in isolation (CUDA events, L2 flushed between runs).

    python -m odin_infer_b200.csrc.microbench gemm --m 8 --n 24576 --k 4096 [--mode 1 --bn 16 --split 3]
    python -m odin_infer_b200.csrc.microbench gemm --m 2048 --n 24576 --k 4096 --pair
    python -m odin_infer_b200.csrc.microbench decode-attention --batch 64 --ctx 640
    python -m odin_infer_b200.csrc.microbench prefill-attention --tokens 2048
    python -m odin_infer_b200.csrc.microbench add-rmsnorm --rows 8 --width 4096 --split 4
    python -m odin_infer_b200.csrc.microbench mma-rate

Prints one JSON line: the median time and the achieved bytes/s and flop/s of the kernel's
algorithmic traffic and work.  Small enough to run under a profiler.  `mma-rate` is of another kind:
it times no kernel of a step but tcgen05.mma itself (see mma_probe.cu), in cycles of the SM clock,
for the shapes and issue orders of the attention kernels, one line per case.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from . import ops

DEV = "cuda:0"


def timeit(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)  # larger than the 126 MB L2
    times = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2]


def paged(batch: int, ctx: int, n_kv: int, hd: int):
    pages_per = (ctx + 63) // 64
    total = batch * pages_per
    perm = torch.randperm(total).to(torch.int32).view(batch, pages_per).to(DEV)
    k = torch.randn(total, n_kv, 64, hd, device=DEV).bfloat16()
    v = torch.randn(total, n_kv, 64, hd, device=DEV).bfloat16()
    return k, v, perm


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=["gemm", "decode-attention", "prefill-attention", "add-rmsnorm", "head-prep", "mma-rate"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--mode", type=int, default=-1, help="-1: as the runtime chooses")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--split", type=int, default=0, help="0: as the runtime chooses")
    ap.add_argument("--stages", type=int, default=0, help="gemm: length of the ring of stages (0: as many as fit)")
    ap.add_argument("--staged", type=int, default=-1,
                    help="gemm, mode 1: K blocks of a CTA's first item staged in tensor memory (-1: as the runtime chooses)")
    ap.add_argument("--pair", action="store_true", help="gemm: the two-CTA kernel (tiles of 256 x 256 on pairs of SMs)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=640)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--width", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args(argv)
    out: dict = {"kernel": args.kernel}

    if args.kernel == "gemm":
        from ..engine.runtime import choose_k_split
        M, N, K = args.m, args.n, args.k
        a = torch.randn(M, K, device=DEV).bfloat16()
        w = torch.randn(N, K, device=DEV).bfloat16()
        if args.pair:
            c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
            ms = timeit(lambda: ops.gemm_tc2(a, w, c), args.iters)
            ops.gemm_tc_check()
            out.update(m=M, n=N, k=K, pair=True, us=round(ms * 1e3, 2), tflops=round(2 * M * N * K / ms / 1e9, 1))
            print(json.dumps(out))
            return 0
        mode = args.mode if args.mode >= 0 else (1 if M <= 128 else 0)
        bn = args.bn or ((16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128) if mode == 1 else 256)
        split = args.split or (choose_k_split((N + 127) // 128, (K + 63) // 64, M) if mode == 1 else 1)
        split = ops.gemm_tc_splits(K, split)
        c = torch.empty((split, M, N) if split > 1 else (M, N), device=DEV,
                        dtype=torch.float32 if split > 1 else torch.bfloat16)
        from ..engine.runtime import STAGED_BLOCKS
        staged = args.staged if args.staged >= 0 else (STAGED_BLOCKS if mode == 1 and bn <= 32 else 0)
        ms = timeit(lambda: ops.gemm_tc(a, w, c, mode, bn, split, args.stages, staged), args.iters)
        ops.gemm_tc_check()
        out.update(m=M, n=N, k=K, mode=mode, bn=bn, split=split, staged=staged, us=round(ms * 1e3, 2),
                   weight_gbs=round(N * K * 2 / ms / 1e6, 1), tflops=round(2 * M * N * K / ms / 1e9, 1))
    elif args.kernel == "decode-attention":
        B, hq, hkv, hd = args.batch, args.heads, args.kv_heads, args.head_dim
        k, v, bt = paged(B, args.ctx, hkv, hd)
        q = torch.randn(B, hq * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        pos = torch.full((B,), args.ctx - 1, dtype=torch.int32, device=DEV)
        seq = torch.arange(B, dtype=torch.int32, device=DEV)
        from ..engine.runtime import decode_key_splits
        n_split = args.split or decode_key_splits(B, hkv, args.ctx)
        scratch = torch.empty(ops.attention_decode_scratch(B, hq, hd, n_split), device=DEV)
        ms = timeit(lambda: ops.attention_decode(q, o, hq, hkv, hd, k, v, pos, seq, bt, 0, scratch, n_split), args.iters)
        out.update(batch=B, ctx=args.ctx, n_split=n_split, us=round(ms * 1e3, 2),
                   kv_gbs=round(2 * B * args.ctx * hkv * hd * 2 / ms / 1e6, 1))
    elif args.kernel == "prefill-attention":
        T, hq, hkv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
        k, v, bt = paged(1, T, hkv, hd)
        q = torch.randn(T, hq * hd, device=DEV).bfloat16()
        o = torch.empty_like(q)
        ss = torch.tensor([0, T], dtype=torch.int32, device=DEV)
        sl = torch.tensor([T], dtype=torch.int32, device=DEV)
        ms = timeit(lambda: ops.attention_prefill(q, o, 1, T, hq, hkv, hd, k, v, ss, sl, bt, 0),
                    args.iters)
        ops.attention_prefill_check()
        out.update(tokens=T, us=round(ms * 1e3, 2), tflops=round(4 * hq * hd * (T * (T + 1) / 2) / ms / 1e9, 1))
    elif args.kernel == "mma-rate":
        # (name, pattern, N, B MN-major, commits per group, CTAs per SM, arithmetic cycles at 4,096 multiply-adds a cycle and SM)
        cases = [("A and B from shared memory, N 64", 0, 64, False, 0, 1, 32),
                 ("A and B from shared memory, N 128", 0, 128, False, 0, 1, 64),
                 ("A and B from shared memory, N 256", 0, 256, False, 0, 1, 128),
                 ("A from tensor memory, N 64", 1, 64, False, 0, 1, 32),
                 ("A from tensor memory, N 128, B MN-major", 1, 128, True, 0, 1, 64),
                 ("two CTAs: A and B from shared memory, N 64", 0, 64, False, 0, 2, 32),
                 ("two CTAs: A from tensor memory, N 128, B MN-major", 1, 128, True, 0, 2, 64),
                 ("page of 64 keys (4 P V + 8 scores N 64)", 2, 0, False, 0, 1, 512),
                 ("page of 64 keys, one commit per group", 2, 0, False, 1, 1, 512),
                 ("page of 64 keys, two commits per group", 2, 0, False, 2, 1, 512),
                 ("two CTAs: page of 64 keys", 2, 0, False, 0, 2, 512),
                 ("two CTAs: page of 64 keys, one commit per group", 2, 0, False, 1, 2, 512),
                 ("two CTAs: page of 64 keys, two commits per group", 2, 0, False, 2, 2, 512),
                 ("two pages (8 P V + 8 scores N 128)", 3, 0, False, 0, 1, 1024),
                 ("two pages, one commit per group", 3, 0, False, 1, 1, 1024),
                 ("two CTAs: two pages, one commit per group", 3, 0, False, 1, 2, 1024),
                 ("eight P V MMAs (N 128), a commit and the wait for it", 4, 0, False, 0, 1, 512),
                 ("eight score MMAs (N 64), a commit and the wait for it", 5, 0, False, 0, 1, 256),
                 ("two CTAs: eight P V MMAs (N 128), a commit and the wait for it", 4, 0, False, 0, 2, 512)]
        for name, pattern, n, b_mn, commits, per_sm, arith in cases:
            iters = 4096 if pattern <= 1 else 512
            best, issue = min(ops.mma_probe(pattern, n, b_mn, commits, per_sm, iters) for _ in range(3))
            line = {"kernel": "mma-rate", "case": name, "cycles": round(best, 1),
                    "unit": "per MMA" if pattern <= 1 else "per step of a CTA", "arithmetic": arith}
            if pattern >= 4:
                line["cycles_until_issued"] = round(issue, 1)
            print(json.dumps(line))
        return 0
    elif args.kernel == "head-prep":
        # the prompt's head preparation: per-head norm of q and k, rotation, cache write, from a bfloat16 projection
        T, hq, hkv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
        k, v, bt = paged(1, T, hkv, hd)
        width = (hq + 2 * hkv) * hd
        qkv = torch.randn(T, width, device=DEV).bfloat16()
        q_out = torch.empty(T, hq * hd, device=DEV, dtype=torch.bfloat16)
        qn = torch.ones(hd, device=DEV).bfloat16()
        ang = torch.rand(T, hd // 2, device=DEV)
        cos, sin = torch.cos(ang), torch.sin(ang)
        pos = torch.arange(T, dtype=torch.int32, device=DEV)
        seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        ms = timeit(lambda: ops.head_prep(qkv, hq, hkv, hd, qn, qn, 1e-6, cos, sin, hd, pos, seq, bt, k, v, write_kv=True,
                                          q_out=q_out), args.iters)
        out.update(tokens=T, us=round(ms * 1e3, 2), gbs=round(2 * T * width * 2 / ms / 1e6, 1))
    else:
        n, d, s = args.rows, args.width, max(args.split, 1)
        x = torch.randn(n, d, device=DEV)
        delta = torch.randn(s, n, d, device=DEV)
        w = torch.ones(d, device=DEV).bfloat16()
        h = torch.empty(n, d, device=DEV, dtype=torch.bfloat16)
        ms = timeit(lambda: ops.add_rmsnorm(x, delta, w, 1e-6, h), args.iters)
        out.update(rows=n, width=d, split=s, us=round(ms * 1e3, 2),
                   gbs=round(n * d * (4 * (s + 2) + 2) / ms / 1e6, 1))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())

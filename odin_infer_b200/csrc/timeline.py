"""Timeline of one replayed decode step: when every kernel's CTAs start, when its wait for the kernel
before it ends ("go": that kernel has completed), and the marks that some kernels set inside.

    ODIN_KERNEL_TRACE=1 python -m odin_infer_b200.csrc.timeline [--batch 8] [--layers 3] [--prompt 512]

Needs the trace build of the kernel libraries (ODIN_KERNEL_TRACE=1 compiles them beside the ordinary ones:
thread 0 of every CTA records %globaltimer into a buffer; see common.cuh).  A tuning tool: the numbers it
prints include the marks' own cost (a few tenths of a microsecond per kernel).
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys


def main(argv=None) -> int:
    if os.environ.get("ODIN_KERNEL_TRACE", "0") in ("", "0"):
        print("timeline: set ODIN_KERNEL_TRACE=1 (the trace build of the kernels records the marks)", file=sys.stderr)
        return 2
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--blocks", type=int, default=0, metavar="GRID",
                    help="also print, block by block, the marks of the first kernel of the last layer whose grid has this size")
    args = ap.parse_args(argv)
    import numpy as np
    import torch
    from .. import Engine, Engine_Opts, StepEntry
    from ..config import config_from_dict
    from . import build

    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=args.hidden, intermediate_size=args.intermediate,
               num_hidden_layers=args.layers, num_attention_heads=args.heads, num_key_value_heads=args.kv_heads,
               head_dim=128, vocab_size=args.vocab, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False)
    engine = Engine.random(config_from_dict(raw), 5, Engine_Opts(max_ctx=4096, max_tokens=args.batch * 1024,
                                                                 max_batch=args.batch, dtype="bfloat16", verbose=False))
    rng = np.random.default_rng(1)
    slots = [engine.take_slot() for _ in range(args.batch)]
    engine.step([StepEntry(s, rng.integers(0, 1000, args.prompt).tolist(), [args.prompt - 1]) for s in slots])

    def step():
        engine.step([StepEntry(s, [5], [0]) for s in slots])
    for _ in range(6):
        step()
    torch.cuda.synchronize()
    cap = 1 << 18
    buf = torch.zeros(1 + 2 * cap, dtype=torch.int64, device="cuda")
    for lib in build._loaded.values():
        f = getattr(lib, "odin_trace_attach", None)
        if f is not None:
            f.argtypes = [ctypes.c_void_p, ctypes.c_uint]
            f(ctypes.c_void_p(buf.data_ptr()), ctypes.c_uint(cap))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    buf.zero_()
    torch.cuda.synchronize()
    step()
    torch.cuda.synchronize()
    h = buf.cpu().numpy()
    n = int(h[0])
    t = h[1:1 + 2 * n:2].astype(np.uint64)
    w = h[2:2 + 2 * n:2].astype(np.uint64)
    point = (w >> np.uint64(56)).astype(int)
    bdim = ((w >> np.uint64(44)) & np.uint64(0xfff)).astype(int)
    grid = ((w >> np.uint64(22)) & np.uint64(0x3fffff)).astype(int)
    blk = (w & np.uint64(0x3fffff)).astype(int)
    us = (t - t.min()).astype(np.int64) / 1000.0
    # kernels in order of their first CTA's start; a kernel is told by (grid, block size), a new one of the same
    # signature begins when a block number comes again
    kernels, open_k = [], {}
    for i in np.argsort(t, kind="stable"):
        sig = (int(grid[i]), int(bdim[i]))
        k = open_k.get(sig)
        if point[i] == 0:
            if k is None or blk[i] in k["seen"]:
                k = {"sig": sig, "seen": set(), "start": [], "go": [], "marks": {}}
                kernels.append(k)
                open_k[sig] = k
            k["seen"].add(blk[i])
            k["start"].append(us[i])
            k.setdefault("by_block", {}).setdefault(int(blk[i]), {})[0] = us[i]
        elif point[i] == 1:
            for kk in kernels:
                if kk["sig"] == sig and blk[i] in kk["seen"] and blk[i] not in kk.setdefault("went", set()):
                    kk["went"].add(blk[i])
                    kk["go"].append(us[i])
                    break
        elif k is not None:
            k["marks"].setdefault(int(point[i]), []).append(us[i])
            k.setdefault("by_block", {}).setdefault(int(blk[i]), {})[int(point[i])] = us[i]
    names = {2: "first item's MMAs issued / loads back / heads prepared", 3: "last commit / sum known / pages multiplied",
             4: "stores issued / end / warps merged", 5: "last tile stored / splits met", 6: "all loads requested"}
    print(f"records {n}; batch {args.batch}, {args.layers} layers; times in us from the step's first mark")
    print("go: the kernel's wait for the kernel before it has ended; 'previous took': from the previous kernel's go to this one's,")
    print("i.e. what the kernel in the line above cost the chain")
    print(f"{'grid':>6} {'thr':>5} | {'first start':>11} {'last start':>10} | {'go':>8} | previous took | marks after go (min..max)")
    prev = None
    for k in kernels:
        if not k["go"]:
            continue
        go = min(k["go"])
        extra = "; ".join(f"{names.get(p, p)}: {min(v) - go:.1f}..{max(v) - go:.1f}" for p, v in sorted(k["marks"].items()))
        print(f"{k['sig'][0]:6d} {k['sig'][1]:5d} | {min(k['start']):11.2f} {max(k['start']):10.2f} | {go:8.2f} | "
              f"{(go - prev) if prev is not None else 0.0:6.2f} | {extra}")
        prev = go
    if args.blocks:
        picked = [k for k in kernels if k["sig"][0] == args.blocks and k.get("go") and k.get("by_block")]
        if picked:
            k = picked[-2] if len(picked) > 1 else picked[-1]  # the last one of the size is the head when the sizes agree
            go = min(k["go"])
            print(f"blocks of the kernel with grid {args.blocks} that went at {go:.2f}: block: mark=us after go ... (0: the block's start)")
            for b in sorted(k["by_block"]):
                print(f"{b:5d}: " + " ".join(f"{p}={v - go:.1f}" for p, v in sorted(k["by_block"][b].items())))
    return 0


if __name__ == "__main__":
    sys.exit(main())

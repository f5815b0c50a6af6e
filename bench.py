#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of the whole batch (default: 8 sequences, 512-token
prompts, context cap 4096).  Prints ONE JSON line:
  value    decoded tokens per second, timed on the device with CUDA events over
           exactly K steps after W warm-up steps (synthetic token ids fed from
           the host each step, no read-back inside the timed region);
  e2e      the same through the Python entry point Engine.generate: host token
           lists in, host token lists out, a device-to-host read every step;
  prefill  one 2,048-token prompt in one step;
  roofline the decode step against the HBM copy bandwidth: every weight it uses
           once plus the live requests' cache, divided by its time;
  points   decode at batch 1 and 64.
Peaks come from MEASURED_PEAKS.json beside this file when it exists.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Qwen3-8B shape
SHAPE_8B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)
WEIGHT_SEED = 5
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        clocks = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        maxes = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "reasons": reasons, "samples": len(clocks)}


def count_params(cfg, n_layers):
    d, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (qd + 2 * kvd) + qd * d + 3 * d * I
    return per_layer, V * d  # layer matrices; head (the embedding table is read by rows only)


def decode_bytes(cfg, n_layers, batch, ctx_tokens):
    """Bytes a decode step has to read: every matrix once (bfloat16) and the live cache."""
    per_layer, head = count_params(cfg, n_layers)
    weights = 2 * (per_layer * n_layers + head)
    kv = 2 * 2 * n_layers * cfg["num_key_value_heads"] * cfg["head_dim"] * ctx_tokens * batch
    return weights + kv


def prefill_flops(cfg, n_layers, T):
    per_layer, head = count_params(cfg, n_layers)
    gemm = 2 * T * per_layer * n_layers + 2 * head  # logits at the last place only
    attn = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2) * n_layers
    return gemm + attn


def run_decode(engine, batch, steps, warmup, vocab, seed=1):
    """Device-timed decode: returns (tokens/s, ms/step, mean context length, kernel launches)."""
    import numpy as np
    import torch
    from odin_infer_b200 import StepEntry
    from odin_infer_b200.csrc import ops
    rng = np.random.default_rng(seed)
    slots = [engine.take_slot() for _ in range(batch)]
    try:
        prompts = [rng.integers(0, vocab, PROMPT).tolist() for _ in range(batch)]
        engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        feed = rng.integers(0, vocab, (warmup + steps, batch))
        for i in range(warmup):
            engine.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
        torch.cuda.synchronize()
        ctx0 = engine.cache.lengths[slots[0]]
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(warmup, warmup + steps):
            engine.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = ops.launch_count() - launches0
        mean_ctx = ctx0 + (steps + 1) / 2
        return batch * steps / (ms / 1e3), ms / steps, mean_ctx, launches
    finally:
        for s in slots:
            engine.give_back_slot(s)


def run_prefill(engine, vocab, reps=3):
    import numpy as np
    import torch
    from odin_infer_b200 import StepEntry
    rng = np.random.default_rng(7)
    best = None
    for r in range(reps + 1):
        toks = rng.integers(0, vocab, PREFILL_TOKENS).tolist()
        slot = engine.take_slot()
        try:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            engine.step([StepEntry(slot, toks, [len(toks) - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        finally:
            engine.give_back_slot(slot)
        if r > 0:  # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def run_e2e(engine, batch, steps, vocab):
    """Through Engine.generate: host token lists in and out, one read-back per step.  Returns the statistics of a
    call of `steps` decode steps and, when that is short, of one of 256 steps as well: the first ~20 decode steps
    after a prompt step run 12 to 15 % slower than the later ones (the prompt step runs at the power cap and the
    SM clock takes ~80 ms to come back), so a short call measures mostly that."""
    import numpy as np
    from odin_infer_b200 import GenerationStats
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, vocab, PROMPT).tolist() for _ in range(batch)]
    engine.generate(prompts, max_new_tokens=4, temperature=0.0, stop_token_ids=[])  # warm-up (graphs, allocator)
    stats = GenerationStats()
    out = engine.generate(prompts, max_new_tokens=steps + 1, temperature=0.0, stop_token_ids=[], stats=stats)
    assert all(len(o.tokens) == steps + 1 for o in out)
    steady = None
    if steps < 128:
        steady = GenerationStats()
        engine.generate(prompts, max_new_tokens=257, temperature=0.0, stop_token_ids=[], stats=steady)
    return stats, steady


SHAPE_1P7B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=2048, intermediate_size=6144, num_hidden_layers=28,
                  num_attention_heads=16, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                  rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960)
SHAPE_32B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                 num_attention_heads=64, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
                 rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960)


def other_workload(which: str) -> int:
    """BASELINE.json configs[3] and configs[4]; one JSON line each, device-timed unless said otherwise."""
    import time

    import numpy as np
    import torch
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine.generate import GenerationStats
    peaks, peak_source = load_peaks()
    if which == "1.7b-mixed":
        raw = dict(SHAPE_1P7B)
        rng = np.random.default_rng(11)
        lens = rng.integers(16, 2049, 64)
        prompts = [rng.integers(0, raw["vocab_size"], int(n)).tolist() for n in lens]
        need = sum((int(n) + 128 + 63) // 64 * 64 for n in lens)
        e = Engine.random(config_from_dict(raw), 6, Engine_Opts(max_ctx=4096, max_tokens=need, max_batch=64,
                                                                dtype="bfloat16", verbose=False))
        e.generate(prompts, max_new_tokens=128, stop_token_ids=[])  # warm-up: the same requests once (kernels, graphs)
        st = GenerationStats()
        t0 = time.perf_counter()
        e.generate(prompts, max_new_tokens=128, stop_token_ids=[], stats=st)
        total = time.perf_counter() - t0
        out = {"metric": "Qwen3-1.7B shape, bf16: 64 prompts of 16..2048 tokens in one batch, 128 new tokens each, "
                         "through Engine.generate (host clock, second pass over the same requests)", "prompt_tokens": int(lens.sum()),
               "ttft_ms": round(st.ttft_s * 1e3, 1), "prefill_tokens_per_s": round(float(lens.sum()) / st.ttft_s),
               "decode_tokens_per_s": round(st.decode_tokens_per_s), "total_s": round(total, 3), "batches": st.n_batches}
    else:
        raw = dict(SHAPE_32B)
        e = Engine.random(config_from_dict(raw), 7, Engine_Opts(max_ctx=8192, max_tokens=8 * 8192, max_batch=8,
                                                                dtype="bfloat16", verbose=False))
        rng = np.random.default_rng(12)
        L = raw["num_hidden_layers"]
        out = {"metric": "Qwen3-32B shape, bf16, 64 layers: a 2,048-token prompt; decoding at context 8192", "peak_source": peak_source}
        for _ in range(3):
            s = e.take_slot()
            p = rng.integers(0, raw["vocab_size"], 2048).tolist()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            e.step([StepEntry(s, p, [2047])])
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
            e.give_back_slot(s)
        out["prefill"] = {"tokens": 2048, "ms": round(ms, 2), "value": round(2048 / ms * 1e3),
                          "frac": round(prefill_flops(raw, L, 2048) / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        for B in (1, 8):
            slots = [e.take_slot() for _ in range(B)]
            ctx0 = 8192 - 72
            for a0 in range(0, ctx0, 2048):  # the context, in pieces of 2,048 tokens
                n = min(2048, ctx0 - a0)
                e.step([StepEntry(s, rng.integers(0, raw["vocab_size"], n).tolist(), []) for s in slots])
            feed = rng.integers(0, raw["vocab_size"], (72, B))
            for i in range(8):
                e.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
            torch.cuda.synchronize()
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(8, 72):
                e.step([StepEntry(s, [int(feed[i, b])], [0]) for b, s in enumerate(slots)])
            b2.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b2) / 64
            out[f"decode_b{B}"] = {"ms_per_step": round(ms, 3), "value": round(B / ms * 1e3, 1), "context": 8192 - 32,
                                   "hbm_frac": round(decode_bytes(raw, L, B, 8192 - 32) / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
            for s in slots:
                e.give_back_slot(s)
    ops.gemm_tc_check()
    ops.attention_prefill_check()
    ops.attention_decode_check()
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-graphs", action="store_true", help="launch the decode step's kernels one by one (for profilers)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end run (for profilers)")
    ap.add_argument("--workload", default="8b", choices=["8b", "1.7b-mixed", "32b-long"],
                    help="8b: the contract's run (default).  The others are further workloads of the baseline's list and "
                         "print a line of their own: 1.7b-mixed = Qwen3-1.7B shape, 64 prompts of 16..2048 tokens, 128 new "
                         "tokens each; 32b-long = Qwen3-32B shape, a 2,048-token prompt, decoding 1 and 8 sequences at context 8192")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is written in Odin (CPU) and Metal (macOS GPU); this image has no Odin compiler, "
                          "it is no Python package, and it has no batched or CUDA path to run"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)
    if args.workload != "8b":
        return other_workload(args.workload)

    import torch
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops

    cfg_raw = dict(SHAPE_8B)
    full_layers = cfg_raw["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg_raw["num_hidden_layers"] = n_layers
    cfg = config_from_dict(cfg_raw)
    peaks, peak_source = load_peaks()
    vocab = cfg_raw["vocab_size"]

    max_batch = 64 if not args.no_points else args.batch
    need = PROMPT + max(warmup, 32) + args.steps + 8
    max_tokens = max(max_batch * ((need + 63) // 64 * 64), ((PREFILL_TOKENS + 63) // 64) * 64)
    engine = Engine.random(cfg, WEIGHT_SEED, Engine_Opts(max_ctx=CONTEXT, max_tokens=max_tokens, max_batch=max_batch,
                                                         dtype="bfloat16", verbose=False,
                                                         cuda_graphs=not args.no_graphs))

    sampler = ClockSampler()
    sampler.start()
    tps, ms_step, mean_ctx, launches = run_decode(engine, args.batch, args.steps, warmup, vocab)
    clocks = sampler.stop()
    ops.gemm_tc_check()
    ops.attention_prefill_check()
    ops.attention_decode_check()

    bytes_step = decode_bytes(cfg_raw, n_layers, args.batch, mean_ctx)
    achieved = bytes_step / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_source}

    if args.no_e2e:
        e2e = None
    else:
        stats, steady = run_e2e(engine, args.batch, args.steps, vocab)
        e2e = {"value": round(stats.decode_tokens_per_s, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": int(engine.last_step_h2d_bytes), "d2h_bytes_per_step": 4 * args.batch,
               "ttft_ms": round(stats.ttft_s * 1e3, 2), "steps": args.steps}
        if steady is not None:
            e2e["value_at_256_steps"] = round(steady.decode_tokens_per_s, 1)

    out = {
        "metric": "decode tokens/s (Qwen3-8B shape, bf16, batch %d, 512-token prompts)" % args.batch,
        "value": round(tps, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (uniform random token ids, random weights N(0,0.02) seed 5)",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": n_layers, "layers_of_config": full_layers,
                   "hidden": cfg_raw["hidden_size"], "q_heads": cfg_raw["num_attention_heads"],
                   "kv_heads": cfg_raw["num_key_value_heads"], "head_dim": cfg_raw["head_dim"],
                   "intermediate": cfg_raw["intermediate_size"], "vocab": vocab, "global_batch": args.batch,
                   "prompt_len": PROMPT, "seq_len": CONTEXT, "decode_ctx_mean": round(mean_ctx, 1),
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (%.1f GB read per step)" % (bytes_step / 1e9),
                   "cuda_graphs": not args.no_graphs},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
    }
    if not args.no_points:
        ms_pf = run_prefill(engine, vocab)
        flops = prefill_flops(cfg_raw, n_layers, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (ms_pf / 1e3), 1), "tokens": PREFILL_TOKENS,
                          "ms": round(ms_pf, 3), "frac": round(flops / (ms_pf / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        pts = {}
        for b in (1, 64):
            # The prompt step of 64 x 512 tokens runs for 0.4 s at the power cap, and the SM clock needs ~80 ms of
            # decoding to come back: at least 32 untimed steps, so that the point is the steady decode rate.
            t, m, c, _ = run_decode(engine, b, min(args.steps, 128), max(warmup, 32), vocab, seed=b)
            pts[f"decode_b{b}"] = round(t, 1)
            pts[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg_raw, n_layers, b, c) / (m / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        out["points"] = pts
        ops.gemm_tc_check()
        ops.attention_prefill_check()
        ops.attention_decode_check()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())

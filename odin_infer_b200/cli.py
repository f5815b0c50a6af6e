"""Command line: token ids in, token ids out.

    python -m odin_infer_b200 <model_dir> --prompt-ids 1,2,3 [flags]

The flags keep the reference CLI's letters and meanings where it has them
(docs/ENVIRONMENT.md:50-62): -t temperature (default 0.6), -p top-p (0.95),
-s seed (0: from the clock), -x repetition penalty (1.0: off), -r print tokens
per second, -f print time to first token, -c max context.  The reference's -j
(threads) and -g (Metal) have no meaning on this engine and are accepted and
ignored; -m (multi-turn) and -k (thinking) belong to its chat template, which
this library (token ids in, token ids out) does not have.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="odin_infer_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    ap.add_argument("--random-config", metavar="CONFIG.JSON",
                    help="no model folder: random weights for this config.json (see --weights-seed)")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--write-random-model", metavar="DIR",
                    help="write config.json and model.safetensors of the random model to DIR and exit")
    src = ap.add_argument_group("prompts (token ids)")
    src.add_argument("--prompt-ids", action="append", default=[], metavar="1,2,3", help="one prompt; may be repeated")
    src.add_argument("--prompt-file", metavar="FILE", help="one prompt per line, ids separated by commas or spaces")
    src.add_argument("--random-prompts", metavar="N:LEN", help="N prompts of LEN uniform random ids (seed 1)")
    ap.add_argument("-n", "--max-new-tokens", type=int, default=256, help="reference default: 256")
    ap.add_argument("-t", dest="temperature", type=float, default=0.6, help="temperature; 0 = greedy")
    ap.add_argument("-p", dest="top_p", type=float, default=0.95, help="top-p; <=0 or >=1 = off")
    ap.add_argument("-s", dest="seed", type=int, default=0, help="RNG seed; 0 = from the clock")
    ap.add_argument("-x", dest="repetition_penalty", type=float, default=1.0, help="repetition penalty; 1.0 = off")
    ap.add_argument("-r", dest="print_tps", action="store_true", help="print decode tokens per second")
    ap.add_argument("-f", dest="print_ttft", action="store_true", help="print time to first token")
    ap.add_argument("-c", dest="max_ctx", type=int, default=4096, help="max context (reference default 4096)")
    ap.add_argument("-j", dest="threads", type=int, default=None, help="ignored (CPU threads of the reference)")
    ap.add_argument("-g", dest="metal", type=int, default=None, help="ignored (Metal switch of the reference)")
    ap.add_argument("--stop-ids", default=None, metavar="7,9", help="stop token ids (default: the config's eos_token_id; '' = none)")
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--json", action="store_true", help="print one JSON object per request instead of id lists")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .config import config_from_dict, load_config
    from .weights import write_random_model

    config = None
    if args.random_config:
        with open(args.random_config) as f:
            config = config_from_dict(json.load(f), args.random_config)
    if args.write_random_model:
        if config is None:
            print("--write-random-model needs --random-config", file=sys.stderr)
            return 2
        write_random_model(args.write_random_model, config, args.weights_seed)
        print(args.write_random_model)
        return 0
    if config is None and not args.model:
        print("give a model folder or --random-config", file=sys.stderr)
        return 2
    for flag, val in (("-j", args.threads), ("-g", args.metal)):
        if val is not None:
            print(f"note: {flag} has no meaning on this engine and is ignored", file=sys.stderr)

    prompts = [parse_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    vocab = (config or load_config(args.model)).to_dict().get("vocab_size", 0)
    if args.random_prompts:
        import numpy as np
        n, length = (int(v) for v in args.random_prompts.split(":"))
        rng = np.random.default_rng(1)
        prompts += [rng.integers(0, vocab, length).tolist() for _ in range(n)]
    if not prompts:
        print("no prompt given (--prompt-ids, --prompt-file or --random-prompts)", file=sys.stderr)
        return 2

    from .engine import Engine, Engine_Opts, GenerationStats
    opts = Engine_Opts(max_ctx=args.max_ctx, max_batch=args.max_batch, dtype=args.dtype, device=args.device)
    engine = Engine.random(config, args.weights_seed, opts) if config is not None else Engine.load(args.model, opts)
    seed = args.seed if args.seed != 0 else time.time_ns() & 0xFFFFFFFF
    stops = None if args.stop_ids is None else parse_ids(args.stop_ids)
    stats = GenerationStats()
    results = engine.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                              top_p=args.top_p, seed=seed, stop_token_ids=stops,
                              repetition_penalty=args.repetition_penalty, stats=stats)
    for i, r in enumerate(results):
        if args.json:
            print(json.dumps({"request": i, "tokens": r.tokens, "finish_reason": r.finish_reason,
                              "prompt_tokens": r.prompt_tokens}))
        else:
            print(",".join(str(t) for t in r.tokens))
    if args.print_ttft:
        print(f"ttft: {stats.ttft_s * 1e3:.1f} ms", file=sys.stderr)
    if args.print_tps:
        print(f"decode: {stats.decode_tokens_per_s:.1f} tok/s ({stats.decode_tokens} tokens, {stats.n_steps} steps, "
              f"{stats.n_batches} batch(es))", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

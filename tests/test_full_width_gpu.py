"""The engine at the real layer sizes (hidden 4096, 32 q / 8 kv heads of 128, intermediate
12288, vocabulary 151936; two layers, random weights) against the plain implementation:
the true 32-bit path and the serving kernels (tcgen05 products with their split-K and SwiGLU
variants, tensor-core attention for prompts and decoding, CUDA graphs), each request whole,
with its last 32 tokens one by one, and in batches of unequal lengths; logits at sampled
positions (the head is 1.2 GFLOP a row).  In 32-bit the cuts must agree bit for bit."""
import numpy as np
import pytest
import torch

from tests import tiny, traces

pytestmark = pytest.mark.gpu

WIDE = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
            rms_norm_eps=1e-6, tie_word_embeddings=False)
SEED = 5
LENGTHS = (70, 161, 300)


def wanted_positions(n: int) -> list[int]:
    """16 places of a request of n tokens: its ends, the borders of cache pages, and places
    that the one-by-one schedule decodes."""
    fixed = {0, 1, n - 1, n - 2, n - 31, n - 32, n - 33, 63, 64, 65, 127, 128, 129, 255, 256, 257}
    picked = sorted(p for p in fixed if 0 <= p < n)
    rng = np.random.default_rng(n)
    while len(picked) < 16:
        p = int(rng.integers(0, n))
        if p not in picked:
            picked = sorted(picked + [p])
    return picked[:16] if n - 1 in picked[:16] else picked[:15] + [n - 1]


@pytest.fixture(scope="module")
def case():
    """Requests, wanted places and the plain implementation's logits there (float32 on the CPU, on the
    very weights the engine generates from the seed: the generator gives the same bits on host and device)."""
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import model_param_specs, random_weights
    from tests.plain import qwen3_plain
    cfg = config_from_dict(WIDE)
    w = random_weights(model_param_specs(cfg), SEED, torch.bfloat16, "cuda:0")
    w = {k: v.to("cpu").float() for k, v in w.items()}
    torch.cuda.empty_cache()
    reqs = {f"r{i}": tiny.random_tokens(n, WIDE["vocab_size"], 300 + i) for i, n in enumerate(LENGTHS)}
    wanted = {rid: wanted_positions(len(t)) for rid, t in reqs.items()}
    refs = {rid: qwen3_plain.forward_whole(WIDE, w, toks, positions=wanted[rid]).double().numpy()
            for rid, toks in reqs.items()}
    del w
    return reqs, wanted, refs


def run(dtype, recs):
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine.trace import replay
    n = traces.max_live_tokens(recs)
    e = Engine.random(config_from_dict(WIDE), SEED, Engine_Opts(max_ctx=n, max_tokens=n, dtype=dtype, verbose=False))
    try:
        got = traces.collect_places(recs, replay(e, recs))
        torch.cuda.synchronize()
        if dtype == "bfloat16":
            ops.gemm_tc_check()
            ops.attention_prefill_check()
            ops.attention_decode_check()
        e.cache.check()
        return got
    finally:
        e.destroy()


def schedules(reqs, wanted):
    return {"whole": traces.restrict(traces.whole(reqs), wanted),
            "last 32 one by one": traces.restrict(traces.tail_one_by_one(reqs, 32), wanted),
            "unequal batch": traces.restrict(traces.batches(reqs, 3, first_part=lambda n: max(1, n - 40)), wanted)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_against_the_plain_implementation(case, dtype):
    reqs, wanted, refs = case
    results = {}
    for what, recs in schedules(reqs, wanted).items():
        got = results[what] = run(dtype, recs)
        for rid, places in wanted.items():
            assert sorted(got[rid]) == places, (what, rid)
            for i, pos in enumerate(places):
                err = tiny.rel_err(got[rid][pos], refs[rid][i])
                assert err <= tiny.TOL[dtype], f"{what} {dtype}: request {rid} position {pos}: {err:.3e}"
    if dtype == "float32":
        # every kernel of the 32-bit path sums in an order that the shapes fix, never the batch: the cuts agree exactly
        for what in ("last 32 one by one", "unequal batch"):
            for rid, places in wanted.items():
                for pos in places:
                    assert np.array_equal(results[what][rid][pos], results["whole"][rid][pos]), \
                        f"float32: '{what}' differs from 'whole' at request {rid} position {pos}"
    else:
        # the greedy token agrees with the plain implementation's wherever its margin is not within rounding
        for rid, places in wanted.items():
            for i, pos in enumerate(places):
                top2 = np.sort(refs[rid][i])[-2:]
                if top2[1] - top2[0] > 4 * tiny.TOL[dtype] * np.abs(refs[rid][i]).max():
                    assert results["whole"][rid][pos].argmax() == refs[rid][i].argmax()

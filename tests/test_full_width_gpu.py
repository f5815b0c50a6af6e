"""The serving kernels at the real layer sizes (hidden 4096, 32 q / 8 kv heads of 128,
intermediate 12288, vocabulary 151936; two layers, random weights): the bfloat16 engine
(tcgen05 products with their split-K and SwiGLU variants, tensor-core attention for prompts
and decoding, CUDA graphs) against the true 32-bit engine on the same weights.  The 32-bit
path itself is checked against the plain implementation on the tiny configurations."""
import numpy as np
import pytest

from tests import tiny

pytestmark = pytest.mark.gpu

WIDE = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
            num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6,
            rms_norm_eps=1e-6, tie_word_embeddings=False)


def run_engine(dtype, prompts, n_decode, feed):
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.config import config_from_dict
    e = Engine.random(config_from_dict(WIDE), 5, Engine_Opts(max_ctx=1024, max_batch=len(prompts), dtype=dtype, verbose=False))
    slots = [e.take_slot() for _ in prompts]
    rows = [e.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).float().cpu().numpy()]
    for i in range(n_decode):
        rows.append(e.step([StepEntry(s, [int(feed[i][b])], [0]) for b, s in enumerate(slots)]).float().cpu().numpy())
    from odin_infer_b200.csrc import ops
    if dtype == "bfloat16":
        ops.gemm_tc_check()
        ops.attention_prefill_check()
        ops.attention_decode_check()
    for s in slots:
        e.give_back_slot(s)
    e.cache.check()
    e.destroy()
    return np.stack(rows)  # [1 + n_decode, B, V]


def test_bfloat16_kernels_agree_with_float32_at_full_width():
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, WIDE["vocab_size"], n).tolist() for n in (1, 130, 300, 64)]
    feed = rng.integers(0, WIDE["vocab_size"], (5, len(prompts)))
    ref = run_engine("float32", prompts, 5, feed)
    got = run_engine("bfloat16", prompts, 5, feed)
    assert not np.isnan(got).any()
    worst = 0.0
    for step in range(ref.shape[0]):
        for b in range(ref.shape[1]):
            err = tiny.rel_err(got[step, b], ref[step, b].astype(np.float64))
            worst = max(worst, err)
            assert err <= tiny.TOL["bfloat16"], f"step {step}, sequence {b}: {err:.3e}"
    # the greedy token agrees wherever the 32-bit margin is not within rounding
    for step in range(ref.shape[0]):
        for b in range(ref.shape[1]):
            top2 = np.sort(ref[step, b])[-2:]
            if top2[1] - top2[0] > 4 * worst * np.abs(ref[step, b]).max():
                assert got[step, b].argmax() == ref[step, b].argmax()

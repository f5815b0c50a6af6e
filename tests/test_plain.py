"""Known-answer tests of the plain implementation (the oracle has to be right first)."""
import math

import torch

from tests.plain import qwen3_plain as P
from tests import tiny


def test_rmsnorm_known():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = P.rmsnorm(x, w, 0.0)
    r = 1.0 / math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[2 * 3 * r, 0.5 * 4 * r]], dtype=torch.float64))


def test_rope_position_zero_is_identity_and_norm_preserving():
    cos, sin = P.rope_tables(5, 8, 10000.0, torch.float64)
    v = torch.randn(5, 3, 8, dtype=torch.float64)
    out = P.rope(v, cos, sin)
    assert torch.allclose(out[0], v[0])
    assert torch.allclose(out.norm(dim=-1), v.norm(dim=-1))
    # pair (i, i + half) at position 1, i = 0 rotates by angle 1
    e = torch.zeros(2, 1, 8, dtype=torch.float64)
    e[1, 0, 0] = 1.0
    o = P.rope(e, cos[:2], sin[:2])
    assert abs(o[1, 0, 0] - math.cos(1.0)) < 1e-7 and abs(o[1, 0, 4] - math.sin(1.0)) < 1e-7


def test_softmax_uniform_and_attention_single_key():
    s = torch.zeros(1, 4, dtype=torch.float64)
    assert torch.allclose(P.softmax_rows(s), torch.full((1, 4), 0.25, dtype=torch.float64))
    q = torch.randn(1, 4, 8, dtype=torch.float64)
    k = torch.randn(1, 2, 8, dtype=torch.float64)
    v = torch.randn(1, 2, 8, dtype=torch.float64)
    o = P.causal_attention(q, k, v).reshape(1, 4, 8)
    assert torch.allclose(o[0, 0], v[0, 0]) and torch.allclose(o[0, 1], v[0, 0])
    assert torch.allclose(o[0, 2], v[0, 1]) and torch.allclose(o[0, 3], v[0, 1])


def test_attention_is_causal_and_window_cuts():
    torch.manual_seed(0)
    q, k, v = (torch.randn(6, 2, 4, dtype=torch.float64) for _ in range(3))
    full = P.causal_attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0  # the future of token 3
    assert torch.allclose(P.causal_attention(q, k2, v2)[:4], full[:4])
    win = P.causal_attention(q, k, v, window=2)
    k3, v3 = k.clone(), v.clone()
    k3[:4], v3[:4] = 5.0, 5.0  # outside the window of token 5
    assert torch.allclose(P.causal_attention(q, k3, v3, window=2)[5], win[5])
    assert not torch.allclose(win[5], full[5])


def test_tied_head_is_embedding_product(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, 0)
    cfg, w = P.read_model_folder(folder, torch.float64)
    assert "lm_head.weight" not in w
    toks = tiny.random_tokens(7, 256, 1)
    logits = P.forward_whole(cfg, w, toks)
    assert logits.shape == (7, 256)
    # the same weights with an explicit head give the same logits
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    assert torch.equal(P.forward_whole(cfg, w2, toks), logits)


def test_prefix_invariance_of_plain(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_B, 2)
    cfg, w = P.read_model_folder(folder, torch.float64)
    toks = tiny.random_tokens(30, 384, 3)
    a = P.forward_whole(cfg, w, toks)
    b = P.forward_whole(cfg, w, toks[:11])
    assert torch.allclose(a[:11], b, atol=1e-12)


def test_float32_and_float64_plain_agree(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_B, 2)
    toks = tiny.random_tokens(40, 384, 3)
    a = tiny.plain_logits(folder, toks, torch.float64)
    b = tiny.plain_logits(folder, toks, torch.float32)
    assert tiny.rel_err(b, a) < 1e-5


def test_sampler_pieces():
    logits = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert P.argmax_first(logits.tolist()) == 1
    p = P.temperature_probs(logits.double(), 0.5)
    assert abs(float(p.sum()) - 1) < 1e-12
    assert P.sample_mult(p.tolist(), 0.0) == 0
    assert P.sample_mult(p.tolist(), 0.999999) == 3 or P.sample_mult(p.tolist(), 0.999999) == 2
    keep = P.top_p_keep(p, 0.6)
    assert keep <= {1, 2} and len(keep) >= 1
    pen = P.repetition_penalty(torch.tensor([1.0, -1.0, 3.0]), [0, 1, 1], 2.0)
    assert pen.tolist() == [0.5, -2.0, 3.0]


import pytest


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_two_independent_restatements_of_the_reference_agree(tmp_path, name):
    """The whole-sequence restatement (torch, matrix products) against the token-by-token one (numpy,
    the reference's own loop structure with key and value arrays): float64 rounding apart, the same
    logits at every position.  The oracle of the GPU tests therefore rests on two readings."""
    import numpy as np
    from tests.plain import qwen3_stepwise as S
    raw, seed = tiny.TINIES[name]
    folder = tiny.make_folder(tmp_path, raw, seed)
    cfg, w = P.read_model_folder(folder, torch.float64)
    toks = tiny.random_tokens(14 if raw["vocab_size"] > 500 else 20, raw["vocab_size"], 40)
    whole = P.forward_whole(cfg, w, toks).numpy()
    steps = S.logits_token_by_token(cfg, {k: v.numpy() for k, v in w.items()}, toks)
    assert steps.shape == whole.shape
    assert tiny.rel_err(steps, whole) < 1e-12

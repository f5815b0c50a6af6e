"""Generation through the Python entry point against the plain implementation: greedy
tokens, long decoding across pages, first tokens, stop tokens, batches one after another,
temperature sampling that does not depend on the batch."""
import numpy as np
import pytest
import torch

from tests import tiny
from tests.plain import qwen3_plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen_models")
    return {name: tiny.make_folder(root, raw, seed) for name, (raw, seed) in tiny.TINIES.items()}


def engine_for(folder, dtype, **kw):
    from odin_infer_b200 import Engine, Engine_Opts
    opts = dict(max_ctx=512, max_batch=4, dtype=dtype, verbose=False)
    opts.update(kw)
    return Engine.load(folder, Engine_Opts(**opts))


def check_greedy(folder, prompts, outs, margin):
    """Teacher-forced on the engine's tokens: each must be the plain argmax, or within
    `margin` (relative to the largest logit) of it, so that a rounding-level tie cannot fail."""
    cfg, w = qwen3_plain.read_model_folder(folder, torch.float64)
    exact = total = 0
    for p, o in zip(prompts, outs):
        ref = qwen3_plain.forward_whole(cfg, w, p + o.tokens)
        for i, tok in enumerate(o.tokens):
            row = ref[len(p) - 1 + i]
            gap = float(row.max() - row[tok])
            assert gap <= margin * float(row.abs().max()), f"token {i}: chose {tok}, plain argmax {int(row.argmax())}, gap {gap:.3e}"
            exact += int(tok == int(row.argmax()))
            total += 1
    return exact / total


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_greedy_generation_matches_plain(folders, name, dtype, margin):
    vocab = tiny.TINIES[name][0]["vocab_size"]
    prompts = [tiny.random_tokens(n, vocab, 200 + n) for n in (5, 11, 17, 1, 70, 40, 23)]
    e = engine_for(folders[name], dtype, max_batch=3)
    outs = e.generate(prompts, max_new_tokens=8, temperature=0.0, stop_token_ids=[])
    e.cache.check()
    assert all(len(o.tokens) == 8 and o.finish_reason == "length" for o in outs)
    frac = check_greedy(folders[name], prompts, outs, margin)
    assert frac >= (1.0 if dtype == "float32" else 0.9)
    e.destroy()


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-5), ("bfloat16", 3e-2)])
def test_long_decoding_across_pages(folders, dtype, margin):
    """150 decoded tokens from a prompt that ends just before a page boundary."""
    vocab = tiny.TINY_B["vocab_size"]
    prompts = [tiny.random_tokens(60, vocab, 1), tiny.random_tokens(3, vocab, 2)]
    e = engine_for(folders["B"], dtype)
    outs = e.generate(prompts, max_new_tokens=150, temperature=0.0, stop_token_ids=[])
    assert [len(o.tokens) for o in outs] == [150, 150]
    check_greedy(folders["B"], prompts, outs, margin)
    e.destroy()


def test_stop_tokens_and_context_limit(folders):
    vocab = tiny.TINY_B["vocab_size"]
    prompts = [tiny.random_tokens(n, vocab, 300 + n) for n in (9, 30)]
    e = engine_for(folders["B"], "float32")
    free = e.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    stop = free[0].tokens[4]
    first = free[0].tokens.index(stop)
    outs = e.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[stop])
    assert outs[0].tokens == free[0].tokens[:first] and outs[0].finish_reason == "stop"
    if stop not in free[1].tokens:
        assert outs[1].tokens == free[1].tokens and outs[1].finish_reason == "length"
    # the configuration's own eos ids are the default stop tokens
    assert e.default_stop_token_ids() == (7, 9)
    e.destroy()
    e = engine_for(folders["B"], "float32", max_ctx=64, max_tokens=128)
    out = e.generate([tiny.random_tokens(60, vocab, 5)], max_new_tokens=50, temperature=0.0, stop_token_ids=[])
    assert len(out[0].tokens) == 4 and out[0].finish_reason == "length"   # 60 + 4 = the context limit
    e.cache.check()
    e.destroy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_composition_does_not_change_tokens(folders, dtype):
    """Greedy and sampled tokens of a request are the same alone, in a batch, and in a later
    batch that reuses slots and pages (bfloat16: same bucket, so same kernels and same sums)."""
    vocab = tiny.TINY_A["vocab_size"]
    prompts = [tiny.random_tokens(n, vocab, 400 + n) for n in (5, 11, 17, 33, 8)]
    e = engine_for(folders["A"], dtype, max_batch=5)
    together = e.generate(prompts, max_new_tokens=10, temperature=0.0, stop_token_ids=[])
    e2 = engine_for(folders["A"], dtype, max_batch=2)
    in_pairs = e2.generate(prompts, max_new_tokens=10, temperature=0.0, stop_token_ids=[])
    if dtype == "float32":
        assert [o.tokens for o in together] == [o.tokens for o in in_pairs]
    # temperature sampling: request i draws from its own stream
    a = e.generate(prompts, max_new_tokens=10, temperature=0.8, seed=4, stop_token_ids=[])
    b = e.generate(prompts, max_new_tokens=10, temperature=0.8, seed=4, stop_token_ids=[])
    c = e.generate(prompts, max_new_tokens=10, temperature=0.8, seed=5, stop_token_ids=[])
    assert [o.tokens for o in a] == [o.tokens for o in b]
    assert [o.tokens for o in a] != [o.tokens for o in c]
    if dtype == "float32":
        alone = e2.generate(prompts[:1], max_new_tokens=10, temperature=0.8, seed=4, stop_token_ids=[])
        assert alone[0].tokens == a[0].tokens
    e.cache.check()
    e2.cache.check()
    e.destroy()
    e2.destroy()


def test_sampled_tokens_follow_the_plain_distribution(folders):
    """First sampled token of one prompt, many seeds: frequencies against the plain softmax."""
    vocab = tiny.TINY_A["vocab_size"]
    prompt = tiny.random_tokens(9, vocab, 77)
    e = engine_for(folders["A"], "float32", max_batch=64, max_tokens=64 * 64)
    counts = np.zeros(vocab)
    for seed in range(12):
        outs = e.generate([prompt] * 64, max_new_tokens=1, temperature=1.5, seed=seed, stop_token_ids=[])
        for o in outs:
            counts[o.tokens[0]] += 1
    ref = tiny.plain_logits(folders["A"], prompt)[-1]
    p = np.exp(ref / 1.5 - (ref / 1.5).max())
    p /= p.sum()
    n = counts.sum()
    # total variation distance between empirical and exact distribution over 768 draws of 256 tokens
    assert 0.5 * np.abs(counts / n - p).sum() < 0.25
    e.destroy()


def test_reference_style_api(folders):
    """engine_load / engine_forward / engine_config as in the reference: one token at a position."""
    from odin_infer_b200 import Engine_Opts, engine_config, engine_destroy, engine_forward, engine_load, StepError
    e = engine_load(folders["A"], Engine_Opts(max_ctx=128, dtype="float32", verbose=False))
    assert engine_config(e).hidden_size == 64
    toks = tiny.random_tokens(6, 256, 9)
    ref = tiny.plain_logits(folders["A"], toks)
    for pos, t in enumerate(toks):
        row = engine_forward(e, t, pos).cpu().numpy()
        assert tiny.rel_err(row, ref[pos]) < tiny.TOL["float32"]
    with pytest.raises(StepError):
        engine_forward(e, toks[0], 3)          # not the next position
    with pytest.raises(StepError):
        engine_forward(e, 256, 6)              # token out of range
    row0 = engine_forward(e, toks[0], 0).cpu().numpy()   # position 0 starts afresh
    assert tiny.rel_err(row0, ref[0]) < tiny.TOL["float32"]
    engine_destroy(e)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_ahead_equals_the_hosts_pace(folders, dtype):
    """Generation that launches each decode step before the host has read the tokens it continues
    from (the default) against generation that reads every token first: the same tokens and reasons,
    greedy and sampled, with sequences that stop at different steps, end by length, and batches one
    after another; and the cache's bookkeeping is whole afterwards."""
    vocab = tiny.TINY_B["vocab_size"]
    prompts = [tiny.random_tokens(n, vocab, 900 + n) for n in (9, 30, 4, 66, 17, 2, 41)]
    ahead = engine_for(folders["B"], dtype, max_batch=3)
    paced = engine_for(folders["B"], dtype, max_batch=3, run_ahead=False)
    free = paced.generate(prompts, max_new_tokens=14, temperature=0.0, stop_token_ids=[])
    stops = sorted({free[0].tokens[3], free[1].tokens[7], free[4].tokens[0], free[6].tokens[13]})
    for kw in (dict(temperature=0.0, stop_token_ids=[]), dict(temperature=0.0, stop_token_ids=stops),
               dict(temperature=0.0, stop_token_ids=stops, include_stop_token=True),
               dict(temperature=0.9, top_p=0.8, seed=3, stop_token_ids=stops)):
        a = ahead.generate(prompts, max_new_tokens=14, **kw)
        b = paced.generate(prompts, max_new_tokens=14, **kw)
        if dtype == "float32" or kw["temperature"] == 0.0:
            # bfloat16: a sequence that has stopped stays one more step in its batch, which can move
            # the step into another batch bucket; sums then round differently, and a draw near the
            # edge of two tokens' shares may fall on the other side
            assert [(o.tokens, o.finish_reason) for o in a] == [(o.tokens, o.finish_reason) for o in b], kw
        if kw["temperature"] == 0.0:
            assert any(o.finish_reason == "stop" for o in b) == bool(kw["stop_token_ids"])
    for e in (ahead, paced):
        e.cache.check()
        assert all(g.pool.n_held == 0 for g in e.cache.groups.values())
        e.destroy()


def test_load_says_when_a_size_falls_off_a_fast_kernel(folders, capfd):
    """Sizes that config.json allows and a fast kernel does not take run on a slower kernel, correctly;
    the engine says so at load instead of leaving it to a profile."""
    e = engine_for(folders["C"], "bfloat16", verbose=True)          # head size 48, five query heads on one kv head
    err = capfd.readouterr().err
    assert any("head_dim 48 is not 64 or 128" in n for n in e.notes) and "note: attention: head_dim 48" in err
    assert any("no power of two" in n for n in e.notes)
    e.destroy()
    for name in ("D", "E"):                                         # head sizes 64 and 128: nothing to say
        e = engine_for(folders[name], "bfloat16")
        assert e.notes == []
        e.destroy()
    e = engine_for(folders["C"], "float32")                         # the 32-bit path has one kernel per operation
    assert e.notes == []
    e.destroy()

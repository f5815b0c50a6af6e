"""The generation loop's decisions, against a fake engine (no GPU)."""
import pytest

from odin_infer_b200.engine.generate import GenerationStats, generate, plan_batches
from odin_infer_b200.sampling import SamplingParams, XorShift64Star, stream_for


class FakeEngine:
    """Next token = (last token + 1) % vocab; records every call."""

    def __init__(self, max_batch=3, max_ctx=32, capacity_tokens=64 * 6, vocab=50):
        self.max_batch, self.max_ctx, self.capacity, self.vocab = max_batch, max_ctx, capacity_tokens, vocab
        self.free = list(range(7, -1, -1))
        self.held = {}
        self.steps = []
        self.slot_log = []

    def default_stop_token_ids(self):
        return (13,)

    def take_slot(self):
        s = self.free.pop()
        self.held[s] = 0
        self.slot_log.append(("take", s))
        return s

    def give_back_slot(self, s):
        assert s in self.held, "slot given back twice"
        del self.held[s]
        self.free.append(s)
        self.slot_log.append(("back", s))

    def fits(self, lengths):
        return sum((n + 63) // 64 * 64 for n in lengths) <= self.capacity

    def step(self, entries):
        self.steps.append([(e.slot, list(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            assert e.slot in self.held
            self.held[e.slot] += len(e.tokens)
            assert self.held[e.slot] <= self.max_ctx
        return [(e.tokens[-1] + 1) % self.vocab for e in entries]

    def sample(self, logits, samplers, params):
        assert len(logits) == len(samplers)
        return list(logits)


def test_unequal_prompts_stop_tokens_and_early_finish():
    e = FakeEngine()
    prompts = [[1, 2, 3], [10], [20, 21, 22, 23, 24]]
    res = generate(e, prompts, max_new_tokens=5)
    assert res[0].tokens == [4, 5, 6, 7, 8] and res[0].finish_reason == "length"
    assert res[1].tokens == [11, 12] and res[1].finish_reason == "stop"   # 13 stops; not emitted
    assert res[2].tokens == [25, 26, 27, 28, 29] and res[2].finish_reason == "length"
    # one prompt step with all three, whole prompts, logits at each prompt's end
    assert e.steps[0] == [(0, [1, 2, 3], [2]), (1, [10], [0]), (2, [20, 21, 22, 23, 24], [4])]
    # the stopped sequence leaves; the others go on by one token each; the stop token is never fed
    assert [len(s) for s in e.steps[1:]] == [3, 3, 2, 2]
    assert all(len(t) == 1 for s in e.steps[1:] for _, t, _ in s)
    assert all(13 not in t for s in e.steps for _, t, _ in s)
    # the last sampled token of a sequence is not run through the model
    assert len(e.steps) == 1 + 4
    assert not e.held


def test_stop_token_can_be_included_and_overridden():
    e = FakeEngine()
    res = generate(e, [[10]], max_new_tokens=8, include_stop_token=True)
    assert res[0].tokens == [11, 12, 13] and res[0].finish_reason == "stop"
    res = generate(e, [[10]], max_new_tokens=4, stop_token_ids=[12])
    assert res[0].tokens == [11] and res[0].finish_reason == "stop"
    res = generate(e, [[10]], max_new_tokens=4, stop_token_ids=[])
    assert res[0].tokens == [11, 12, 13, 14]
    res = generate(e, [[12]], max_new_tokens=4)            # the very first sampled token stops
    assert res[0].tokens == [] and res[0].finish_reason == "stop"


def test_context_limit_ends_a_sequence():
    e = FakeEngine(max_ctx=8)
    res = generate(e, [[20, 21, 22, 23, 24]], max_new_tokens=100, stop_token_ids=[])
    assert res[0].tokens == [25, 26, 27] and res[0].finish_reason == "length"  # 5 + 3 = 8 = the limit
    with pytest.raises(ValueError, match="no room"):
        generate(e, [[1] * 8], max_new_tokens=1)
    with pytest.raises(ValueError, match="empty prompt"):
        generate(e, [[]], max_new_tokens=1)


def test_batches_one_after_another_reuse_slots():
    e = FakeEngine(max_batch=2)
    prompts = [[i] for i in (1, 20, 30, 40, 2)]
    stats = GenerationStats()
    res = generate(e, prompts, max_new_tokens=3, stats=stats)
    assert [r.tokens for r in res] == [[2, 3, 4], [21, 22, 23], [31, 32, 33], [41, 42, 43], [3, 4, 5]]
    assert stats.n_batches == 3 and stats.prefill_tokens == 5
    takes = [s for op, s in e.slot_log if op == "take"]
    assert takes == [0, 1, 1, 0, 0] or sorted(set(takes)) == [0, 1]   # only two slots ever used
    assert not e.held
    # decode tokens: every sampled token after a sequence's first
    assert stats.decode_tokens == 5 * 2


def test_plan_batches_by_count_and_capacity():
    assert plan_batches([5, 5, 5, 5, 5], 3, 2, lambda l: True) == [[0, 1], [2, 3], [4]]
    fits = lambda lens: sum((n + 63) // 64 for n in lens) <= 4
    assert plan_batches([100, 100, 10, 200, 1], 28, 8, fits) == [[0, 1], [2], [3], [4]] or \
        plan_batches([100, 100, 10, 200, 1], 28, 8, fits) == [[0, 1], [2, 3], [4]]
    # a request that does not fit even alone still gets a batch of its own (the engine then reports it)
    assert plan_batches([1000], 10, 8, lambda l: False) == [[0]]


def test_slots_given_back_when_a_step_fails():
    e = FakeEngine()
    calls = {"n": 0}
    real = e.step

    def failing(entries):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("boom")
        return real(entries)
    e.step = failing
    with pytest.raises(RuntimeError, match="boom"):
        generate(e, [[1], [2]], max_new_tokens=10, stop_token_ids=[])
    assert not e.held


def test_rng_is_the_reference_generator():
    # xorshift64* by hand for one step (sampler/sampler.odin:68-77)
    s = 0x123456789ABCDEF
    x = s
    x ^= x >> 12
    x ^= (x << 25) & (2 ** 64 - 1)
    x ^= x >> 27
    expect = ((x * 0x2545F4914F6CDD1D) & (2 ** 64 - 1)) >> 32
    g = XorShift64Star(s)
    assert g.random_u32() == expect
    f = XorShift64Star(s).random_f32()
    assert f == (expect >> 8) / 16777216.0 and 0 <= f < 1
    # seed 0 is usable, and streams differ between sequences but not between runs
    a, b = stream_for(0, 0), stream_for(0, 1)
    assert a.state != 0 and a.state != b.state
    assert stream_for(0, 0).random_f32() == a.random_f32()
    assert SamplingParams(repetition_penalty=0.5).repetition_penalty == 1.0


class _Pending:
    def __init__(self, toks):
        self.device_tokens = list(toks)

    def tokens(self):
        return list(self.device_tokens)


class FakeAheadEngine(FakeEngine):
    """The same engine with sampling that leaves the tokens "on the device": the loop then runs one
    step ahead and a step may take its tokens from the last sampling instead of from the host."""

    def step(self, entries, device_tokens=None):
        if device_tokens is not None:
            toks, src = device_tokens
            assert all(e.tokens == [0] for e in entries), "placeholders only"
            entries = [type(e)(e.slot, [toks[src[b] if src is not None else b]], e.want) for b, e in enumerate(entries)]
        return super().step(entries)

    def sample_async(self, logits, samplers, params):
        return _Pending(self.sample(logits, samplers, params))


def test_one_step_ahead_gives_the_same_tokens():
    prompts = [[1, 2, 3], [10], [20, 21, 22, 23, 24], [11], [40]]
    for kwargs in (dict(max_new_tokens=5), dict(max_new_tokens=8, include_stop_token=True),
                   dict(max_new_tokens=1), dict(max_new_tokens=2), dict(max_new_tokens=6, stop_token_ids=[])):
        a, b = FakeEngine(max_batch=3), FakeAheadEngine(max_batch=3)
        ra, rb = generate(a, prompts, **kwargs), generate(b, prompts, **kwargs)
        assert [(r.tokens, r.finish_reason) for r in ra] == [(r.tokens, r.finish_reason) for r in rb], kwargs
        assert not b.held and sorted(b.free) == sorted(a.free)
    # a sequence that ends by length is left out of the step ahead; one that meets a stop token has run
    # one step for nothing (the stop token was fed), and nobody else's tokens changed
    e = FakeAheadEngine()
    res = generate(e, [[10], [30]], max_new_tokens=4)
    assert res[0].tokens == [11, 12] and res[0].finish_reason == "stop"
    assert res[1].tokens == [31, 32, 33, 34] and res[1].finish_reason == "length"
    fed = [[t[0] for _, t, _ in s] for s in e.steps[1:]]
    assert fed == [[11, 31], [12, 32], [13, 33]], fed   # 13 fed once; the step after [34] was never launched
    # the context limit, and the penalty that keeps the loop on the host's pace
    e = FakeAheadEngine(max_ctx=8)
    res = generate(e, [[20, 21, 22, 23, 24]], max_new_tokens=100, stop_token_ids=[])
    assert res[0].tokens == [25, 26, 27] and res[0].finish_reason == "length"
    e = FakeAheadEngine()
    res = generate(e, [[10]], max_new_tokens=4, params=SamplingParams(repetition_penalty=1.3))
    assert all(13 not in t for s in e.steps for _, t, _ in s)


def test_one_step_ahead_stats_and_failures():
    e = FakeAheadEngine(max_batch=2)
    stats = GenerationStats()
    res = generate(e, [[i] for i in (1, 20, 30, 40, 2)], max_new_tokens=3, stats=stats)
    assert [r.tokens for r in res] == [[2, 3, 4], [21, 22, 23], [31, 32, 33], [41, 42, 43], [3, 4, 5]]
    assert stats.n_batches == 3 and stats.decode_tokens == 5 * 2 and not e.held
    e = FakeAheadEngine()
    calls = {"n": 0}
    real = e.step

    def failing(entries, device_tokens=None):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("boom")
        return real(entries, device_tokens)
    e.step = failing
    with pytest.raises(RuntimeError, match="boom"):
        generate(e, [[1], [2]], max_new_tokens=10, stop_token_ids=[])
    assert not e.held

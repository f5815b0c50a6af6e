"""The integer tables of a step (no GPU): what every kernel reads to find a token's sequence,
position and pages; and that the usual decode step, which updates the tables of the step before in
place, leaves exactly what writing them anew would."""
import numpy as np
import pytest

from odin_infer_b200.cache import CacheManager, KVRequest, PAGE
from odin_infer_b200.engine.step import StepBatch, StepEntry, StepError


def manager(window=0):
    m = CacheManager(64 * 40, 64 * 8)
    m.add_entry(KVRequest(2, 16), 0)
    if window:
        m.add_entry(KVRequest(2, 16, window), 0)
    m.entry_writes = [True] * len(m.line_of)
    return m


def tables(b: StepBatch) -> dict:
    out = {k: getattr(b, k).clone().numpy() for k in ("tok_ids", "tok_pos", "tok_seq", "logit_rows", "seq_start",
                                                        "seq_slots", "seq_len_after")}
    for key, bt in b.block_tables.items():
        out[("bt", key)] = bt.clone().numpy()
    return out


def test_start_step_tables():
    m = manager()
    slots = [m.take_slot() for _ in range(3)]
    entries = [StepEntry(slots[0], [5, 6, 7], [2]), StepEntry(slots[1], [9], [0]), StepEntry(slots[2], list(range(70)), [0, 69])]
    starts = [m.extend(e.slot, len(e.tokens)) for e in entries]
    b = StepBatch(m, entries, starts, "cpu", pad_rows_to=80, pad_seqs_to=4)
    t = tables(b)
    assert b.n_seqs == 3 and b.n_tokens == 74 and b.n_rows == 80 and not b.all_single and b.all_start
    assert b.max_new == 80   # padded rows (a captured prompt step): launch shapes hold for any count up to the rows
    assert list(t["tok_ids"][:5]) == [5, 6, 7, 9, 0] and list(t["tok_pos"][:6]) == [0, 1, 2, 0, 0, 1]
    assert list(t["tok_seq"][:5]) == [0, 0, 0, 1, 2] and (t["tok_seq"][74:] == -1).all()   # padding rows
    assert list(t["seq_start"]) == [0, 3, 4, 74, 74] and list(t["seq_len_after"]) == [3, 1, 70, 0]
    assert list(t["logit_rows"]) == [2, 3, 4, 73] and b.wanted_rows == [2, 3, 4, 73]
    bt = next(v for k, v in t.items() if isinstance(k, tuple))
    assert (bt[0, 1:] == -1).all() and bt[0, 0] >= 0 and (bt[2, :2] >= 0).all() and (bt[3] == -1).all()
    assert len({int(bt[0, 0]), int(bt[1, 0]), int(bt[2, 0]), int(bt[2, 1])}) == 4          # no page held twice
    assert StepBatch(m, entries, starts, "cpu").max_new == 70
    with pytest.raises(StepError, match="outside"):
        StepBatch(m, [StepEntry(slots[0], [1], [1])], [3], "cpu")


@pytest.mark.parametrize("window", [0, 128])
def test_decode_steps_in_place_equal_tables_written_anew(window):
    m = manager(window)
    rng = np.random.default_rng(window)
    slots = [m.take_slot() for _ in range(4)]
    lens = [3, 63, 64, 130]
    for s, n in zip(slots, lens):
        m.extend(s, n)
        m.after_step(s)
    graph_like = None
    for step in range(140):                       # across page borders and out of the window
        toks = rng.integers(0, 1000, len(slots)).tolist()
        entries = [StepEntry(s, [t], [0]) for s, t in zip(slots, toks)]
        starts = [m.extend(s, 1) for s in slots]
        if graph_like is None:
            graph_like = StepBatch(m, entries, starts, "cpu", pad_rows_to=8, pad_seqs_to=8, all_rows_wanted=True)
        else:
            graph_like.fill(entries, starts)      # the in-place path
        anew = StepBatch(m, entries, starts, "cpu", pad_rows_to=8, pad_seqs_to=8, all_rows_wanted=True)
        a, b = tables(graph_like), tables(anew)
        for k in a:
            assert np.array_equal(a[k], b[k]), (step, k)
        assert graph_like.max_len_after == anew.max_len_after and graph_like.lengths_after == anew.lengths_after
        for s in slots:
            m.after_step(s)
        if step == 70:                            # a sequence leaves: the next fill is not the usual step
            m.give_back_slot(slots.pop(1))
    m.check()


def test_wanted_rows_follow_each_steps_want_lists():
    """A batch that is refilled in place (a captured decode graph) hands back the rows that THIS
    step's entries want: want lists may change from one one-token step to the next."""
    m = manager()
    slots = [m.take_slot() for _ in range(3)]
    for s in slots:
        m.extend(s, 4)
        m.after_step(s)
    wants = [([0], [0], [0]), ([0], [], [0]), ([], [], []), ([], [0], []), ([0], [0], [0]), ([], [], [0, 0])]
    graph_like = None
    for ws in wants:
        entries = [StepEntry(s, [7], list(w)) for s, w in zip(slots, ws)]
        starts = [m.extend(s, 1) for s in slots]
        if graph_like is None:
            graph_like = StepBatch(m, entries, starts, "cpu", pad_rows_to=4, pad_seqs_to=4, all_rows_wanted=True)
        else:
            graph_like.fill(entries, starts)
        anew = StepBatch(m, entries, starts, "cpu")
        assert graph_like.wanted_rows == anew.wanted_rows == [b for b, w in enumerate(ws) for _ in w]
        for s in slots:
            m.after_step(s)
    entries = [StepEntry(s, [7], [0]) for s in slots]
    entries[1].want = [1]
    starts = [m.extend(s, 1) for s in slots]
    with pytest.raises(StepError, match="outside"):
        graph_like.fill(entries, starts)


def test_fixed_logit_rows_are_rewritten_when_the_wants_move():
    """Without `all_rows_wanted` the logit rows are part of the tables: a one-token step whose
    wants differ from the step before is written anew, or refused if the count changed."""
    m = manager()
    slots = [m.take_slot() for _ in range(2)]
    for s in slots:
        m.extend(s, 2)
        m.after_step(s)
    def step(ws, b=None):
        entries = [StepEntry(s, [3], list(w)) for s, w in zip(slots, ws)]
        starts = [m.extend(s, 1) for s in slots]
        if b is None:
            b = StepBatch(m, entries, starts, "cpu")
        else:
            b.fill(entries, starts)
        for s in slots:
            m.after_step(s)
        return b
    b = step(([0], []))
    assert list(tables(b)["logit_rows"]) == [0]
    step(([], [0]), b)
    assert list(tables(b)["logit_rows"]) == [1] and b.wanted_rows == [1]
    with pytest.raises(StepError, match="number of wanted rows"):
        step(([0], [0]), b)

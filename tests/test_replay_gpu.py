"""The engine against the plain implementation, through trace replay: each request
alone and whole; with its last 32 tokens one by one; in batches of unequal lengths
whose shorter requests end earlier, batch after batch so that slots and pages are
used again.  In 32-bit and in bfloat16, for tiny configurations that differ in
every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import tiny, traces

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 70, 129], "B": [1, 7, 23, 40, 64, 65, 200], "C": [3, 33, 90],
           "D": [1, 63, 64, 65, 130, 300], "E": [2, 40, 128, 257]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: tiny.make_folder(root, raw, seed) for name, (raw, seed) in tiny.TINIES.items()}


@pytest.fixture(scope="module")
def requests_and_refs(folders):
    out = {}
    for name, folder in folders.items():
        vocab = tiny.TINIES[name][0]["vocab_size"]
        reqs = {f"r{i}": tiny.random_tokens(n, vocab, 100 + i) for i, n in enumerate(LENGTHS[name])}
        refs = {rid: tiny.plain_logits(folder, toks) for rid, toks in reqs.items()}
        out[name] = (reqs, refs)
    return out


def run(folder, dtype, recs, graphs=True, collect=traces.collect):
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.engine.trace import replay
    n = traces.max_live_tokens(recs)
    engine = Engine.load(folder, Engine_Opts(max_ctx=n, max_tokens=n, dtype=dtype, verbose=False, cuda_graphs=graphs))
    try:
        results = replay(engine, recs)
        engine.cache.check()
        assert all(g.pool.n_held == 0 for g in engine.cache.groups.values())
        return collect(recs, results)
    finally:
        engine.destroy()


def check(got, refs, dtype, what):
    worst = 0.0
    for rid, ref in refs.items():
        assert got[rid].shape == ref.shape, (what, rid, got[rid].shape, ref.shape)
        for pos in range(ref.shape[0]):
            err = tiny.rel_err(got[rid][pos], ref[pos])
            worst = max(worst, err)
            assert err <= tiny.TOL[dtype], f"{what} {dtype}: request {rid} first differs at position {pos}: {err:.3e}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole(folders, requests_and_refs, name, dtype):
    reqs, refs = requests_and_refs[name]
    check(run(folders[name], dtype, traces.whole(reqs)), refs, dtype, "whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_last_32_one_by_one(folders, requests_and_refs, name, dtype):
    reqs, refs = requests_and_refs[name]
    check(run(folders[name], dtype, traces.tail_one_by_one(reqs, 32)), refs, dtype, "last32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_unequal_batches_slots_reused(folders, requests_and_refs, name, dtype):
    reqs, refs = requests_and_refs[name]
    check(run(folders[name], dtype, traces.batches(reqs, 3)), refs, dtype, "batches of 3")
    check(run(folders[name], dtype, traces.batches(reqs, 2, first_part=lambda n: max(1, n - 5))), refs, dtype,
          "batches of 2")


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_want_lists_that_change_from_step_to_step(folders, requests_and_refs, name, dtype, graphs):
    """One-token steps whose entries want their logits in some steps and not in others (a step may
    want nothing): exactly the wanted places come back, each equal to the plain implementation's."""
    reqs, refs = requests_and_refs[name]
    recs = traces.one_by_one_sparse_wants(reqs, 3)
    got = run(folders[name], dtype, recs, graphs, traces.collect_places)
    asked = {rid: set() for rid in reqs}
    seen = {rid: 0 for rid in reqs}
    for rec in recs:
        for e in rec["entries"]:
            asked[e["id"]] |= {seen[e["id"]] + w for w in e["want"]}
            seen[e["id"]] += len(e["tokens"])
    for rid, ref in refs.items():
        assert set(got.get(rid, {})) == asked[rid], (rid, sorted(got.get(rid, {})), sorted(asked[rid]))
        assert len(ref) - 1 in asked[rid]
        for pos, row in got[rid].items():
            err = tiny.rel_err(row, ref[pos])
            assert err <= tiny.TOL[dtype], f"sparse wants {dtype}: request {rid} position {pos}: {err:.3e}"


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_requests_join_a_running_batch(folders, requests_and_refs, name, dtype, graphs):
    """Steps that mix one-token continuations with whole prompts and pieces of prompts; ends free the
    slots and pages that the joiners take."""
    reqs, refs = requests_and_refs[name]
    check(run(folders[name], dtype, traces.joining(reqs, 3), graphs), refs, dtype, "joining, 3 wide")
    check(run(folders[name], dtype, traces.joining(reqs, 2, tail=20), graphs), refs, dtype, "joining, 2 wide")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_cuts_agree_with_each_other(folders, requests_and_refs, name, dtype):
    """The same position under different cuts.  In 32-bit: the same bits (every kernel of that path
    adds in an order that the shapes fix, never the batch or the cut).  In bfloat16: equal beyond
    rounding, far tighter than the distance to the plain implementation."""
    reqs, _ = requests_and_refs[name]
    a = run(folders[name], dtype, traces.whole(reqs))
    others = {"last 32": run(folders[name], dtype, traces.tail_one_by_one(reqs, 32)),
              "batches": run(folders[name], dtype, traces.batches(reqs, 4)),
              "joining": run(folders[name], dtype, traces.joining(reqs, 3))}
    for what, b in others.items():
        for rid in reqs:
            if dtype == "float32":
                same = (b[rid] == a[rid]).all(axis=1)
                assert same.all(), f"{what}: request {rid} first differs at position {int(np.argmin(same))}"
            else:
                assert tiny.rel_err(b[rid], a[rid].astype(np.float64)) <= 2e-2, (what, rid)


def test_short_prompts_replayed_as_graphs(folders):
    """Prompt steps of up to 1,024 tokens are captured per bucket of rows and of sequences and replayed
    (padding rows of sequence -1, empty padding sequences): the same logits as the eager step, at bucket
    edges, for pieces that continue a sequence, with two wanted places, for a few sequences of unequal
    lengths; a bucket's graph is used again for other lengths."""
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.csrc import ops
    raw, _ = tiny.TINIES["D"]
    out = {}
    for graphs in (False, True):
        e = Engine.load(folders["D"], Engine_Opts(max_ctx=1536, max_tokens=4 * 1536, dtype="bfloat16", verbose=False,
                                                  cuda_graphs=graphs))
        rows = []
        try:
            for i, n in enumerate((2, 31, 32, 33, 64, 65, 100, 129, 300, 1000, 90)):
                s = e.take_slot()
                toks = tiny.random_tokens(n + 40, raw["vocab_size"], 700 + i)
                a = e.step([StepEntry(s, toks[:n], [0, n - 1])])                  # the prompt, two places wanted
                b = e.step([StepEntry(s, toks[n:], [len(toks) - n - 1])])         # a piece of 40 that continues it
                rows += [a.float().cpu(), b.float().cpu()]
                e.give_back_slot(s)
            # a few sequences at once: the same buckets (128 rows, 4 sequences, 3 wanted places), the lengths
            # spread differently each time, the longest beyond what the graph was captured with
            for i, lens in enumerate(((5, 60, 20), (70, 3, 10), (1, 1, 97), (40, 40, 40))):
                slots = [e.take_slot() for _ in lens]
                toks = [tiny.random_tokens(n, raw["vocab_size"], 800 + 10 * i + j) for j, n in enumerate(lens)]
                rows.append(e.step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, toks)]).float().cpu())
                rows.append(e.step([StepEntry(s, [7], [0]) for s in slots]).float().cpu())   # and one token each
                for s in slots:
                    e.give_back_slot(s)
            torch.cuda.synchronize()
            ops.gemm_tc_check()
            ops.attention_prefill_check()
            if graphs:
                keys = [k for k in e.graphs._graphs if k[0] == "prompt"]
                assert len(keys) < 2 * 11, "lengths of one bucket share a graph"
                assert sum(1 for k in keys if k[2] == 4) == 1, "the four steps of three sequences share one graph"
        finally:
            e.destroy()
        out[graphs] = rows
    for a, b in zip(out[True], out[False]):
        assert a.shape == b.shape
        assert (a - b).abs().max().item() <= 2e-2 * b.abs().max().item()


def test_trace_run_program(folders, requests_and_refs, tmp_path):
    """The program itself: JSON lines in, .f32 files and `done` lines out."""
    reqs, refs = requests_and_refs["A"]
    recs = traces.batches(reqs, 3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "out")
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
         "--out", out, "--max-tokens", str(traces.max_live_tokens(recs))],
        input="".join(json.dumps(r) + "\n" for r in recs), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {r['step']}" for r in recs]
    vocab = tiny.TINY_A["vocab_size"]
    results = {r["step"]: np.fromfile(os.path.join(out, f"{r['step']}.f32"), dtype="<f4").reshape(-1, vocab) for r in recs}
    check(traces.collect(recs, results), refs, "float32", "trace_run")

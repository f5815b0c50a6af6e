"""Builders of replay traces and the bookkeeping to read their results back."""
from __future__ import annotations

import numpy as np


def whole(requests: dict[str, list[int]]):
    """Each request alone, its whole sequence in one step, logits everywhere."""
    recs = []
    for i, (rid, toks) in enumerate(requests.items()):
        recs.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return recs


def tail_one_by_one(requests: dict[str, list[int]], tail: int = 32):
    """Each request alone: all but the last `tail` tokens in one step, then one token per step."""
    recs, n = [], 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        recs.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                     "end": [rid] if head == len(toks) else []})
        n += 1
        for p in range(head, len(toks)):
            recs.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                         "end": [rid] if p == len(toks) - 1 else []})
            n += 1
    return recs


def batches(requests: dict[str, list[int]], batch_size: int, first_part=lambda n: n // 2 + 1):
    """Batches that start together with unequal lengths, then go on by one token per
    step; a request ends when its tokens run out, the others go on; batch after batch."""
    recs, n = [], 0
    ids = list(requests)
    for b0 in range(0, len(ids), batch_size):
        group = ids[b0:b0 + batch_size]
        done = {rid: first_part(len(requests[rid])) for rid in group}
        ents = [{"id": rid, "tokens": requests[rid][:done[rid]], "want": list(range(done[rid]))} for rid in group]
        recs.append({"step": n, "entries": ents, "end": [rid for rid in group if done[rid] == len(requests[rid])]})
        n += 1
        live = [rid for rid in group if done[rid] < len(requests[rid])]
        while live:
            ents, end = [], []
            for rid in live:
                ents.append({"id": rid, "tokens": [requests[rid][done[rid]]], "want": [0]})
                done[rid] += 1
                if done[rid] == len(requests[rid]):
                    end.append(rid)
            recs.append({"step": n, "entries": ents, "end": end})
            n += 1
            live = [rid for rid in live if rid not in end]
    return recs


def max_live_tokens(recs, page: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to a page."""
    held: dict[str, int] = {}
    worst = 0
    for rec in recs:
        for e in rec["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum((v + page - 1) // page * page for v in held.values()))
        for rid in rec["end"]:
            held.pop(rid, None)
    return worst


def collect(recs, results: dict) -> dict[str, np.ndarray]:
    """{request id: [positions, vocab]} from per-step result arrays (every position wanted)."""
    rows: dict[str, dict[int, np.ndarray]] = {}
    seen: dict[str, int] = {}
    for rec in recs:
        arr = results.get(rec["step"])
        r = 0
        for e in rec["entries"]:
            base = seen.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], {})[base + w] = arr[r]
                r += 1
            seen[e["id"]] = base + len(e["tokens"])
        assert arr is None or r == arr.shape[0]
    return {rid: np.stack([d[p] for p in sorted(d)]) for rid, d in rows.items()}

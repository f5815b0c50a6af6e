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


def collect_places(recs, results: dict) -> dict[str, dict[int, np.ndarray]]:
    """{request id: {position: logits}} for traces that want only some positions."""
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
        assert (arr is None and r == 0) or r == arr.shape[0], (rec["step"], r, None if arr is None else arr.shape)
    return rows


def one_by_one_sparse_wants(requests: dict[str, list[int]], batch_size: int, head: int = 3):
    """Batches that bring `head` tokens each and then one token per step, with want lists that
    change from step to step: in step n request i of the batch wants its token iff (n + i) % 3 != 0,
    every third step wants nothing at all, and the last place of every request is wanted."""
    recs, n = [], 0
    ids = list(requests)
    for b0 in range(0, len(ids), batch_size):
        group = ids[b0:b0 + batch_size]
        done = {rid: min(head, len(requests[rid])) for rid in group}
        recs.append({"step": n, "entries": [{"id": rid, "tokens": requests[rid][:done[rid]],
                                             "want": [done[rid] - 1] if done[rid] == len(requests[rid]) else []}
                                            for rid in group],
                     "end": [rid for rid in group if done[rid] == len(requests[rid])]})
        n += 1
        live = [rid for rid in group if done[rid] < len(requests[rid])]
        while live:
            ents, end = [], []
            for i, rid in enumerate(live):
                last = done[rid] + 1 == len(requests[rid])
                wanted = last or (n % 3 != 2 and (n + i) % 3 != 0)
                ents.append({"id": rid, "tokens": [requests[rid][done[rid]]], "want": [0] if wanted else []})
                done[rid] += 1
                if last:
                    end.append(rid)
            recs.append({"step": n, "entries": ents, "end": end})
            n += 1
            live = [rid for rid in live if rid not in end]
    return recs


def joining(requests: dict[str, list[int]], width: int = 3, tail: int = 6):
    """Requests that join a running batch: while the live requests go on by one token per step, a
    new one brings its prompt (all but its last `tail` tokens) in the same step, every second
    joiner in two pieces over two steps; a request that ends frees the slot that the next joiner
    takes.  Logits wanted everywhere."""
    recs, n = [], 0
    pending = list(requests)
    live: dict[str, list[int]] = {}    # id -> sizes of the pieces still to feed
    done: dict[str, int] = {}
    joined = 0
    while pending or live:
        if pending and len(live) < width:
            rid = pending.pop(0)
            L = len(requests[rid])
            head = max(1, L - tail)
            pieces = [head] if (joined % 2 == 0 or head < 2) else [head // 2, head - head // 2]
            live[rid] = pieces + [1] * (L - head)
            done[rid] = 0
            joined += 1
        ents, end = [], []
        for rid in list(live):
            k = live[rid].pop(0)
            ents.append({"id": rid, "tokens": requests[rid][done[rid]:done[rid] + k], "want": list(range(k))})
            done[rid] += k
            if not live[rid]:
                end.append(rid)
                del live[rid]
        recs.append({"step": n, "entries": ents, "end": end})
        n += 1
    return recs


def restrict(recs, wanted: dict):
    """The same schedule with logits asked for at the wanted absolute positions only
    (wanted: {request id: positions})."""
    seen: dict = {}
    out = []
    for rec in recs:
        ents = []
        for e in rec["entries"]:
            base = seen.get(e["id"], 0)
            ents.append({"id": e["id"], "tokens": e["tokens"],
                         "want": [w for w in range(len(e["tokens"])) if base + w in wanted[e["id"]]]})
            seen[e["id"]] = base + len(e["tokens"])
        out.append({"step": rec["step"], "entries": ents, "end": rec["end"]})
    return out

"""Trace replay on an engine: the loop behind bin/trace_run.

One record per step: {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.
Requests are told apart by id; an id seen for the first time takes a slot, an id in
`end` gives it back after the step.  Nothing is sampled.
"""
from __future__ import annotations

import os
from typing import Callable, Iterable

from .step import StepEntry


def replay(engine, records: Iterable[dict], out_dir: str | None = None,
           on_done: Callable[[int], None] | None = None) -> dict:
    """Runs the records in order.  Logits of a step in which something is wanted are
    written to out_dir/<step>.f32 (little-endian float32 [wanted, vocab]) when out_dir
    is given, and are returned as numpy arrays by step number in any case."""
    if out_dir is not None:
        os.makedirs(out_dir, exist_ok=True)
    slot_of: dict[str, int] = {}
    results: dict = {}
    try:
        for rec in records:
            step_no = rec["step"]
            entries = []
            for ent in rec.get("entries", []):
                rid = str(ent["id"])
                if rid not in slot_of:
                    slot_of[rid] = engine.take_slot()
                entries.append(StepEntry(slot_of[rid], [int(t) for t in ent["tokens"]],
                                         [int(w) for w in ent.get("want", [])]))
            logits = engine.step(entries) if entries else None
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                if out_dir is not None:
                    arr.tofile(os.path.join(out_dir, f"{step_no}.f32"))
                results[step_no] = arr
            for rid in rec.get("end", []):
                rid = str(rid)
                if rid in slot_of:
                    engine.give_back_slot(slot_of.pop(rid))
            if on_done is not None:
                on_done(step_no)
    finally:
        for slot in slot_of.values():
            engine.give_back_slot(slot)
    return results

"""One step of a batch: the tokens it brings, and everything the kernels need
to find each token's sequence, position and cache pages.

A step is either a start (sequences bring their first tokens, of unequal
number) or a continuation by one token each; continuations by several tokens
are accepted too (a prompt cut in pieces).  Only the tokens given are run.
Padding rows (used to give a replayed CUDA graph a fixed shape) carry sequence
number -1 and are skipped by every kernel that reads or writes the cache.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch


@dataclasses.dataclass
class StepEntry:
    """One sequence's share of a step."""
    slot: int
    tokens: list[int]
    want: list[int] = dataclasses.field(default_factory=list)  # places among `tokens` whose logits are asked for


class StepError(ValueError):
    pass


class StepBatch:
    """Device-side view of a step, handed to every part."""

    def __init__(self, cache, entries: list[StepEntry], start_positions: list[int], device, pad_rows_to: int = 0):
        self.cache = cache
        self.n_seqs = len(entries)
        tok_ids, tok_pos, tok_seq, rows = [], [], [], []
        seq_start = [0]
        for b, (e, p0) in enumerate(zip(entries, start_positions)):
            base = len(tok_ids)
            n = len(e.tokens)
            tok_ids.extend(e.tokens)
            tok_pos.extend(range(p0, p0 + n))
            tok_seq.extend([b] * n)
            seq_start.append(base + n)
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} token(s)")
                rows.append(base + w)
        self.n_tokens = len(tok_ids)
        self.n_rows = max(self.n_tokens, pad_rows_to)
        pad = self.n_rows - self.n_tokens
        tok_ids += [0] * pad
        tok_pos += [0] * pad
        tok_seq += [-1] * pad
        self.all_single = all(len(e.tokens) == 1 for e in entries)
        self.max_new = max((len(e.tokens) for e in entries), default=0)
        self.slots = [e.slot for e in entries]
        self.lengths_after = [p0 + len(e.tokens) for e, p0 in zip(entries, start_positions)]
        self.max_len_after = max(self.lengths_after, default=0)
        self.n_logit_rows = len(rows)

        def dev(a):
            return torch.tensor(a, dtype=torch.int32).to(device, non_blocking=True) if len(a) else \
                torch.zeros(0, dtype=torch.int32, device=device)
        self.tok_ids, self.tok_pos, self.tok_seq = dev(tok_ids), dev(tok_pos), dev(tok_seq)
        self.logit_rows = dev(rows)
        self.seq_start = dev(seq_start)
        self.seq_slots = dev(self.slots)
        self.seq_len_after = dev(self.lengths_after)
        self.block_tables = {}
        for key, g in cache.groups.items():
            bt = np.ascontiguousarray(g.block_table[self.slots]) if self.slots else np.zeros((0, g.max_pages_per_seq), np.int32)
            self.block_tables[key] = torch.from_numpy(bt).to(device, non_blocking=True)

    # ---- what a mixer asks for ------------------------------------------
    def kv(self, entry: int):
        """(keys, values, block table) of the cache line that schedule entry `entry` uses:
        keys/values [page][kv head][64][head_dim], block table int32 [sequences, pages]."""
        line = self.cache.line_of[entry]
        if line is None:
            return None, None, None
        key, idx = line
        g = self.cache.groups[key]
        return g.k[idx], g.v[idx], self.block_tables[key]

    def writes_cache(self, entry: int) -> bool:
        return self.cache.entry_writes[entry]

    def state(self, entry: int) -> torch.Tensor:
        """The fixed-size state of schedule entry `entry`: uint8 [slots, bytes]; row
        `seq_slots[b]` belongs to sequence b of this step."""
        off, n = self.cache.state_offset_of[entry], self.cache.state_bytes_of[entry]
        return self.cache.state[:, off:off + n]

"""One step of a batch: the tokens it brings, and everything the kernels need
to find each token's sequence, position and cache pages.

A step is either a start (sequences bring their first tokens, of unequal
number) or a continuation by one token each; continuations by several tokens
are accepted too (a prompt cut in pieces).  Only the tokens given are run.
Padding rows (they give a replayed CUDA graph a fixed shape) carry sequence
number -1 and are skipped by every kernel that reads or writes the cache.

All integer tables of a step live in one pinned host array and one device array
of the same layout, so a step costs one host-to-device copy; a captured decode
graph keeps its device array and is refilled in place.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..cache.groups import PAGE


@dataclasses.dataclass
class StepEntry:
    """One sequence's share of a step."""
    slot: int
    tokens: list[int]
    want: list[int] = dataclasses.field(default_factory=list)  # places among `tokens` whose logits are asked for


class StepError(ValueError):
    pass


class StepBatch:
    """Device-side view of a step, handed to every part.

    Per token row t (n_rows of them, the first n_tokens real): tok_ids[t], tok_pos[t]
    (position in its sequence), tok_seq[t] (which sequence of this step; -1 padding).
    Per sequence b: seq_slots[b] (its slot: row of the state area), seq_start[b]
    (first token row; n_seqs + 1 entries), seq_len_after[b] (its length once this step
    is done), and one block table row per cache group.  logit_rows: the token rows
    whose logits are wanted.  Host copies for parts that size their launches:
    n_seqs, n_tokens, slots, lengths_after, seq_start_host, all_single, max_new.
    """

    def __init__(self, cache, entries: list[StepEntry], start_positions: list[int], device,
                 pad_rows_to: int = 0, pad_seqs_to: int = 0, all_rows_wanted: bool = False):
        self.cache = cache
        self.device = device
        self.n_seq_cap = max(len(entries), pad_seqs_to)
        self.n_row_cap = max(sum(len(e.tokens) for e in entries), pad_rows_to)
        self.all_rows_wanted = all_rows_wanted
        self._for_graph = pad_rows_to > 0 or pad_seqs_to > 0  # fixed buffers of a captured step
        wanted = sum(len(e.want) for e in entries)
        self.n_logit_cap = self.n_row_cap if all_rows_wanted else wanted
        # layout of the arena (int32 counts)
        off = 0
        self._where: dict[str, tuple[int, tuple[int, ...]]] = {}

        def put(name, *shape):
            nonlocal off
            n = int(np.prod(shape)) if shape else 1
            self._where[name] = (off, shape)
            off += (n + 3) // 4 * 4  # keep every table 16-byte aligned
        put("tok_ids", self.n_row_cap)
        put("tok_pos", self.n_row_cap)
        put("tok_seq", self.n_row_cap)
        put("logit_rows", self.n_logit_cap)
        put("seq_start", self.n_seq_cap + 1)
        put("seq_slots", self.n_seq_cap)
        put("seq_len_after", self.n_seq_cap)
        for key, g in cache.groups.items():
            put(("bt", key), self.n_seq_cap, g.max_pages_per_seq)
        self._host_t = torch.empty(max(off, 4), dtype=torch.int32, pin_memory=(torch.device(device).type == "cuda"))
        self._host = self._host_t.numpy()
        self._dev = torch.empty(max(off, 4), dtype=torch.int32, device=device)

        def view(name):
            o, shape = self._where[name]
            n = int(np.prod(shape)) if shape else 1
            return self._dev[o:o + n].view(*shape)
        self.tok_ids, self.tok_pos, self.tok_seq = view("tok_ids"), view("tok_pos"), view("tok_seq")
        self.logit_rows = view("logit_rows")
        self.seq_start, self.seq_slots, self.seq_len_after = view("seq_start"), view("seq_slots"), view("seq_len_after")
        self.block_tables = {key: view(("bt", key)) for key in cache.groups}
        self._copied = None
        self._host_views: dict = {}
        self.h2d_bytes = self._host_t.numel() * 4
        self.fill(entries, start_positions)

    def _h(self, name):
        v = self._host_views.get(name)
        if v is None:
            o, shape = self._where[name]
            n = int(np.prod(shape)) if shape else 1
            v = self._host_views[name] = self._host[o:o + n].reshape(shape)
        return v

    def fill(self, entries: list[StepEntry], start_positions: list[int]) -> None:
        """(Re)write the tables for these entries and copy them to the device."""
        if self._copied is not None:
            self._copied.synchronize()  # the last copy out of the pinned array must be over before it is rewritten
        if self._advance(entries, start_positions):
            return
        n_tok = sum(len(e.tokens) for e in entries)
        if len(entries) > self.n_seq_cap or n_tok > self.n_row_cap:
            raise StepError("step does not fit the buffers it was built for")
        ids, pos, seq = self._h("tok_ids"), self._h("tok_pos"), self._h("tok_seq")
        ids[:] = 0
        pos[:] = 0
        seq[:] = -1
        starts = self._h("seq_start")
        starts[:] = n_tok
        rows = []
        r = 0
        for b, (e, p0) in enumerate(zip(entries, start_positions)):
            n = len(e.tokens)
            ids[r:r + n] = e.tokens
            pos[r:r + n] = np.arange(p0, p0 + n, dtype=np.int32)
            seq[r:r + n] = b
            starts[b] = r
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} token(s)")
                rows.append(r + w)
            r += n
        self.n_seqs = len(entries)
        self.n_tokens = n_tok
        self.seq_start_host = [int(v) for v in starts[:len(entries)]] + [n_tok]
        self.n_rows = self.n_row_cap
        self.slots = [e.slot for e in entries]
        self.wanted_rows = rows
        lr = self._h("logit_rows")
        if self.all_rows_wanted:
            lr[:] = np.arange(self.n_row_cap, dtype=np.int32)
            self.n_logit_rows = self.n_row_cap
        else:
            if len(rows) != self.n_logit_cap:
                raise StepError("the number of wanted rows changed under fixed buffers")
            lr[:] = rows
            self.n_logit_rows = len(rows)
        sl, la = self._h("seq_slots"), self._h("seq_len_after")
        sl[:] = 0
        la[:] = 0
        sl[:self.n_seqs] = self.slots
        self.lengths_after = [p0 + len(e.tokens) for e, p0 in zip(entries, start_positions)]
        la[:self.n_seqs] = self.lengths_after
        self.all_single = all(len(e.tokens) == 1 for e in entries)
        self.all_start = all(p0 == 0 for p0 in start_positions)
        self.max_new = max((len(e.tokens) for e in entries), default=0)
        if self._for_graph and not self.all_single:
            # rows padded for a captured prompt step: the kernels' shapes must hold for any count of tokens up to the rows
            self.max_new = self.n_row_cap
        self.max_len_after = max(self.lengths_after, default=0)
        for key, g in self.cache.groups.items():
            bt = self._h(("bt", key))
            bt[:] = -1
            if self.slots:
                bt[:self.n_seqs] = g.block_table[self.slots]
        self._last_starts = list(start_positions)
        self._upload()

    def _upload(self) -> None:
        self._dev.copy_(self._host_t, non_blocking=True)
        if self._dev.is_cuda:
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

    def _advance(self, entries: list[StepEntry], start_positions: list[int]) -> bool:
        """The usual decode step: the sequences of the last fill, in the same order, one token
        further each.  Only the token ids, the positions, the lengths and (where a sequence
        entered a new page or a window let pages go) the block tables change; the tables are
        updated in place instead of being written anew.  False if this is not such a step."""
        last = getattr(self, "_last_starts", None)
        if (last is None or not self.all_single or len(entries) != self.n_seqs
                or any(len(e.tokens) != 1 or e.slot != s for e, s in zip(entries, self.slots))
                or any(p != q + 1 for p, q in zip(start_positions, last))):
            return False
        # which logits are wanted may change from step to step: with every row computed
        # (a captured graph) only the list of rows to hand back changes; with fixed logit rows the
        # tables are written anew
        rows = []
        for b, e in enumerate(entries):
            for w in e.want:
                if w != 0:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its 1 token(s)")
                rows.append(b)
        if not self.all_rows_wanted and rows != self.wanted_rows:
            return False
        self.wanted_rows = rows
        n = self.n_seqs
        self._h("tok_ids")[:n] = [e.tokens[0] for e in entries]
        self._h("tok_pos")[:n] += 1
        self._h("seq_len_after")[:n] += 1
        self.lengths_after = [p + 1 for p in start_positions]
        self.max_len_after += 1
        self.all_start = False
        for key, g in self.cache.groups.items():
            if g.request.window > 0 or any(p % PAGE == 0 for p in start_positions):
                self._h(("bt", key))[:n] = g.block_table[self.slots]
        self._last_starts = list(start_positions)
        self._upload()
        return True

    def take_tokens(self, tokens: torch.Tensor, src: list[int] | None) -> None:
        """The step's token ids from the device instead of from the host (one token per sequence):
        sequence b takes tokens[src[b]] (tokens[b] if src is None).  Runs on the stream after the
        copy of the tables, so it is what the step's kernels see."""
        n = self.n_seqs
        if src is None:
            self.tok_ids[:n].copy_(tokens[:n])
        else:
            idx = torch.tensor(src, dtype=torch.int64).to(tokens.device, non_blocking=True)
            self.tok_ids[:n].copy_(tokens.index_select(0, idx))

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

"""Cache groups: storage for the layers that keep the same kind of thing.

A mixer asks for what it keeps per sequence with a `KVRequest` (keys and
values of `n_kv_heads` x `head_dim` per token, all of them or a window of the
last `window`), or with state bytes of fixed size (see state.py).  Layers with
equal requests share one group; every group has storage, a page pool and block
tables of its own.

Storage of one group: K and V as [line][page][kv head][PAGE tokens][head_dim],
one "line" per schedule entry that writes to the group.  A sequence's pages are
listed in its row of the block table, in order of position; page p of a row
holds positions [p*PAGE, (p+1)*PAGE).  In a window group the pages that lie
wholly before the window are given back as the sequence grows (their block
table entries become -1).
"""
from __future__ import annotations

import dataclasses

import numpy as np

from .pages import CacheError, PagePool

PAGE = 64  # tokens per page; the unit in which a request's length is rounded up


@dataclasses.dataclass(frozen=True)
class KVRequest:
    """What an attention-like mixer keeps: keys and values per token."""
    n_kv_heads: int
    head_dim: int
    window: int = 0  # 0: all keys; W > 0: the last W

    @property
    def key(self):
        return ("kv", self.n_kv_heads, self.head_dim, self.window)


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class KVGroup:
    """Host-side bookkeeping of one group; `attach_storage` adds the device tensors."""

    def __init__(self, request: KVRequest, n_lines: int, n_pages: int, max_slots: int, max_pages_per_seq: int):
        self.request = request
        self.n_lines = n_lines
        self.pool = PagePool(n_pages)
        self.max_pages_per_seq = max_pages_per_seq
        self.block_table = np.full((max_slots, max_pages_per_seq), -1, dtype=np.int32)
        self.first_live_page = np.zeros(max_slots, dtype=np.int64)  # window groups: pages before it were released
        self.k = None
        self.v = None

    def storage_shape(self) -> tuple[int, ...]:
        r = self.request
        return (self.n_lines, self.pool.n_pages, r.n_kv_heads, PAGE, r.head_dim)

    def bytes_per_token(self, itemsize: int) -> int:
        r = self.request
        return 2 * self.n_lines * r.n_kv_heads * r.head_dim * itemsize

    def attach_storage(self, k, v) -> None:
        self.k, self.v = k, v

    def grow(self, slot: int, old_len: int, new_len: int) -> None:
        """Make room for positions [old_len, new_len) of `slot`."""
        have, need = pages_for(old_len), pages_for(new_len)
        if need > self.max_pages_per_seq:
            raise CacheError(f"a sequence of {new_len} tokens needs {need} pages; the limit is {self.max_pages_per_seq}")
        if need > have:
            new_pages = self.pool.take(need - have)
            self.block_table[slot, have:need] = new_pages

    def release_before_window(self, slot: int, length: int) -> None:
        """Window groups: give back the pages that no later token can see."""
        w = self.request.window
        if w <= 0:
            return
        # the next query sits at position `length`; it sees keys > length - w
        first_needed = max(0, length - w + 1)
        first_page = first_needed // PAGE
        start = int(self.first_live_page[slot])
        if first_page > start:
            row = self.block_table[slot, start:first_page]
            self.pool.give_back([int(p) for p in row if p >= 0])
            self.block_table[slot, start:first_page] = -1
            self.first_live_page[slot] = first_page

    def release_all(self, slot: int) -> None:
        row = self.block_table[slot]
        self.pool.give_back([int(p) for p in row if p >= 0])
        self.block_table[slot, :] = -1
        self.first_live_page[slot] = 0

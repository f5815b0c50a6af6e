"""The cache of an engine: slots, their lengths, the groups, the state area.

A slot belongs to one sequence from the start of its batch until it ends; it
names the sequence's rows in every group's block table and in the state area.
Slots are given back when a sequence ends and are handed out again; a slot's
state bytes are zeroed when it is handed out (device memory is not zeroed by
itself).  Nothing here touches the device except through `zero_state`.
"""
from __future__ import annotations

from .groups import KVGroup, KVRequest, PAGE, pages_for
from .pages import CacheError


class CacheManager:
    def __init__(self, max_tokens: int, max_seq_len: int, max_slots: int | None = None):
        """max_tokens: the most tokens that live sequences hold together, each
        rounded up to a whole page.  max_seq_len: the longest single sequence."""
        if max_tokens <= 0:
            raise CacheError(f"max_tokens must be positive, got {max_tokens}")
        self.n_pages = pages_for(max_tokens)
        self.max_seq_len = min(max_seq_len, self.n_pages * PAGE)
        self.max_pages_per_seq = pages_for(self.max_seq_len)
        # every live sequence holds at least one page
        self.max_slots = self.n_pages if max_slots is None else min(max_slots, self.n_pages)
        self._free_slots = list(range(self.max_slots - 1, -1, -1))
        self._live = [False] * self.max_slots
        self.lengths = [0] * self.max_slots
        self.groups: dict[tuple, KVGroup] = {}
        self.line_of: list[tuple[tuple, int] | None] = []  # schedule entry -> (group key, line in group)
        self.state_bytes_of: list[int] = []                 # schedule entry -> bytes of fixed-size state
        self.state_offset_of: list[int] = []
        self.state_bytes_per_slot = 0
        self.state = None  # device tensor [max_slots, state_bytes_per_slot] uint8, attached by the engine
        self.zero_state = None  # callable(slot) set by the engine

    # ---- layout, fixed at load time -------------------------------------
    def add_entry(self, kv: KVRequest | None, state_bytes: int, shares_line_of: int | None = None) -> int:
        """Register one schedule entry; returns its index.

        kv: what the entry's mixer keeps per token (None: nothing).
        shares_line_of: index of an earlier entry whose keys and values this one
        reads instead of keeping its own.
        """
        idx = len(self.line_of)
        if shares_line_of is not None:
            if not (0 <= shares_line_of < idx) or self.line_of[shares_line_of] is None:
                raise CacheError(f"schedule entry {idx} reads the cache of entry {shares_line_of}, which keeps none")
            src_key, src_line = self.line_of[shares_line_of]
            if kv is not None and kv.key != src_key:
                raise CacheError(f"schedule entry {idx} cannot read the cache of entry {shares_line_of}: "
                                 f"it wants {kv.key}, the other keeps {src_key}")
            self.line_of.append((src_key, src_line))
        elif kv is not None:
            g = self.groups.get(kv.key)
            if g is None:
                g = KVGroup(kv, 0, self.n_pages, self.max_slots, self.max_pages_per_seq)
                self.groups[kv.key] = g
            self.line_of.append((kv.key, g.n_lines))
            g.n_lines += 1
        else:
            self.line_of.append(None)
        # states are 256-byte aligned within a slot's row
        self.state_bytes_of.append(state_bytes)
        self.state_offset_of.append(self.state_bytes_per_slot)
        self.state_bytes_per_slot += (state_bytes + 255) // 256 * 256
        return idx

    # ---- slots ------------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def take_slot(self) -> int:
        if not self._free_slots:
            raise CacheError(f"no free slot: all {self.max_slots} are held")
        s = self._free_slots.pop()
        self._live[s] = True
        self.lengths[s] = 0
        if self.state_bytes_per_slot and self.zero_state is not None:
            self.zero_state(s)
        return s

    def give_back_slot(self, slot: int) -> None:
        self._check_live(slot)
        for g in self.groups.values():
            g.release_all(slot)
        self._live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def _check_live(self, slot: int) -> None:
        if not (0 <= slot < self.max_slots):
            raise CacheError(f"slot {slot} is out of range (0..{self.max_slots - 1})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is not held (given back twice, or never taken)")

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and self._live[slot]

    # ---- growth -----------------------------------------------------------
    def can_hold(self, extra_tokens_per_slot: dict[int, int]) -> bool:
        need = 0
        for slot, extra in extra_tokens_per_slot.items():
            need += pages_for(self.lengths[slot] + extra) - pages_for(self.lengths[slot])
        return all(need <= g.pool.n_free for g in self.groups.values()) if self.groups else True

    def extend(self, slot: int, n_tokens: int) -> int:
        """Reserve room for n_tokens more tokens of `slot`; returns its old length."""
        self._check_live(slot)
        old = self.lengths[slot]
        new = old + n_tokens
        if new > self.max_seq_len:
            raise CacheError(f"slot {slot}: {new} tokens exceed the context limit of {self.max_seq_len}")
        done = []
        try:
            for g in self.groups.values():
                g.grow(slot, old, new)
                done.append(g)
        except CacheError:
            for g in done:  # undo, so that a failed step leaves nothing held
                have, got = pages_for(old), pages_for(new)
                pages = [int(p) for p in g.block_table[slot, have:got] if p >= 0]
                g.pool.give_back(pages)
                g.block_table[slot, have:got] = -1
            raise
        self.lengths[slot] = new
        return old

    def after_step(self, slot: int) -> None:
        """Called when a step's kernels are enqueued: window groups drop dead pages."""
        for g in self.groups.values():
            g.release_before_window(slot, self.lengths[slot])

    def check(self) -> None:
        """Invariants: no page lost or held twice; free slots hold nothing."""
        for g in self.groups.values():
            g.pool.check()
            held = [int(p) for p in g.block_table.flatten() if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError("a page is in two block table entries")
            if len(held) != g.pool.n_held:
                raise CacheError(f"{g.pool.n_held} pages are held but {len(held)} are in block tables")
            for s in range(self.max_slots):
                if not self._live[s] and (g.block_table[s] >= 0).any():
                    raise CacheError(f"free slot {s} still holds pages")
        if len(set(self._free_slots)) != len(self._free_slots):
            raise CacheError("a slot is in the free list twice")
        free_slots = set(self._free_slots)
        for s in range(self.max_slots):
            if self._live[s] == (s in free_slots):
                raise CacheError(f"slot {s} is {'both live and free' if self._live[s] else 'lost'}")

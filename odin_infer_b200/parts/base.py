"""What a part is: the interfaces of mixer, feed-forward, norm, position
encoding, block, embedding and head, and the registries that name them.

A part is built from keyword arguments alone (its sizes, constants and tensor
names); it never learns which model it is in.  A model is a list of blocks
whose parts are chosen layer by layer through `PartSpec(kind, args)`.

Life of a part:
  1. `Part(**args)`                      sizes and names are fixed;
  2. `params()`                          the tensors it wants from the model folder;
  3. `bind(tensors, rt)`                 it takes them (and may fuse or drop them);
  4. `forward(...)`                      once per step, enqueueing kernels on the
                                         current stream; no host synchronisation.

A part that says `graph_safe = True` promises that its `forward` may be captured in a
CUDA graph once and replayed for other steps of the same shape: it reads sequence
numbers, slots, positions and page tables from the step's DEVICE tensors only (the host
copies change between replays), sizes its launches by what holds for every replay
(`step.n_rows` token rows, `step.n_seq_cap` sequences, some of them padding), skips rows
of sequence -1, keeps nothing on the host from one call to the next, and calls nothing
that synchronises or allocates outside torch's stream-ordered allocator.  The default is
False: a model with one such part runs every step eagerly, which is always right.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable

import torch

from ..cache import KVRequest


@dataclasses.dataclass(frozen=True)
class ParamSpec:
    """One tensor of the model folder.

    init: how random-weights mode fills it: "matrix" N(0, 0.02), "norm" 1 + N(0, 0.1),
    "zeros", or "int_table" (int32 zeros).  alias_of: the name of another tensor that
    stands in when this one is absent (a tied head).
    """
    name: str
    shape: tuple[int, ...]
    init: str = "matrix"
    alias_of: str | None = None

    @property
    def is_integer(self) -> bool:
        return self.init == "int_table"


@dataclasses.dataclass(frozen=True)
class PartSpec:
    kind: str
    args: dict = dataclasses.field(default_factory=dict)


class Part:
    """Base of all parts."""

    def params(self) -> list[ParamSpec]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor], rt) -> None:
        pass

    # May this part's forward be captured in a CUDA graph and replayed (see the module's text)?
    graph_safe = False

    def kernel_groups(self) -> set[str]:
        """Kernel libraries this part launches (compiled before the first step)."""
        return set()

    def notes(self, rt) -> list[str]:
        """What a user should know at load about how this part will run with its sizes (a size that
        a fast kernel does not take and what runs instead); printed once, never an error."""
        return []


class ResidualAdded:
    """The answer of `Runtime.linear(..., add_to=x)` when the product has added its result to
    the residual stream x itself (in its epilogue): nothing is left to add.  A block turns it
    into "no pending update" before the next norm sees it."""


class Norm(Part):
    def forward(self, rt, x: torch.Tensor, delta, rows: torch.Tensor | None = None):
        """x: the 32-bit residual stream [n, width], updated in place by `delta`
        (None, [n, width] or [splits, n, width]); returns the normalised rows in
        the runtime's element type.  rows: gather these rows only (x untouched)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, rt, n_positions: int) -> None:
        """Build whatever tables positions [0, n_positions) need."""

    def rotation(self):
        """(cos, sin, rotary_dim) tables [n_positions, rotary_dim/2] of 32-bit floats for
        mixers that rotate q and k, or None."""
        return None

    def on_embedding(self, rt, step, x: torch.Tensor) -> None:
        """Hook for encodings that act on the embedded tokens (in place)."""


class Mixer(Part):
    def cache_request(self) -> KVRequest | None:
        """Keys and values this mixer keeps per token, or None."""
        return None

    def state_bytes(self) -> int:
        """Bytes of fixed-size state this mixer keeps per sequence."""
        return 0

    # A mixer or feed-forward that sets this also takes a keyword `residual=` (the 32-bit
    # residual stream its update is meant for) and may pass it to its last product as
    # `Runtime.linear(..., add_to=residual)`, returning whatever that returns.
    takes_residual = False

    def forward(self, rt, step, h: torch.Tensor, entry: int) -> torch.Tensor:
        """h: [T, width] normalised input.  entry: index of the schedule entry being run
        (names the cache line and the state through `step`).  Returns the update of the
        residual stream, [T, width] or [splits, T, width]."""
        raise NotImplementedError


class FeedForward(Part):
    takes_residual = False  # as for Mixer

    def forward(self, rt, step, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    def forward(self, rt, step, x: torch.Tensor, pending, entry: int):
        """x: residual stream (in place); pending: an update not yet added to it (None, [n, width]
        or [splits, n, width]).  Returns (x, pending)."""
        raise NotImplementedError

    @property
    def mixer(self) -> Mixer:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, rt, step) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, rt, step, h: torch.Tensor) -> torch.Tensor:
        """h: [rows, width] normalised; returns 32-bit logits [rows, vocab]."""
        raise NotImplementedError


# ---------------------------------------------------------------- registries
_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {}, "embedding": {}, "head": {},
}


def register_part(role: str, kind: str):
    """Class decorator: make `kind` buildable wherever a part of `role` is wanted."""
    if role not in _REGISTRIES:
        raise KeyError(f"unknown part role '{role}' (known: {', '.join(_REGISTRIES)})")

    def deco(cls):
        _REGISTRIES[role][kind] = cls
        return cls
    return deco


def build_part(role: str, spec: PartSpec):
    table = _REGISTRIES[role]
    if spec.kind not in table:
        raise KeyError(f"no {role} named '{spec.kind}' is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[spec.kind](**spec.args)

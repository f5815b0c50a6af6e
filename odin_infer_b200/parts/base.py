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

    # True for a part whose forward launches kernels of this package only (through `ops` and the
    # runtime) and calls nothing that would put other work on the stream: only then may the
    # runtime record a decode step's operations and run them as programs of one persistent
    # kernel, where the order of launches is no longer the order of execution for anything else.
    kernels_only = False

    def kernel_groups(self) -> set[str]:
        """Kernel libraries this part launches (compiled before the first step)."""
        return set()


@dataclasses.dataclass
class NormedRows:
    """Rows that a norm has weighted but not yet scaled: row j stands for
    rows[j] / sqrt(sum(ssq[j]) / width + eps).  What a product with a `ResidualSink` hands to
    the norm it was made for; a product that takes it as input applies the factor to its sums
    (`Runtime.linear`), anything else asks the runtime to `materialize` it."""
    rows: torch.Tensor   # [n, width] in the runtime's element type
    ssq: torch.Tensor    # [n, parts] 32-bit shares of the rows' sums of squares
    width: int
    eps: float
    norm: Any            # the norm part these rows are the output of

    @property
    def shape(self):
        return self.rows.shape


@dataclasses.dataclass
class ResidualSink:
    """Where a part's last product may put its result itself: added to the residual stream x,
    and on through `norm` (see `Runtime.linear`).  A part that is handed a sink and cannot use
    it ignores it and returns its update as usual."""
    x: torch.Tensor
    norm: Any


class ResidualAdded:
    """What a product returns that has added its result to the sink's residual stream already:
    nothing is left to add, the norm still has to be taken."""


class Norm(Part):
    def sink(self, x: torch.Tensor) -> ResidualSink | None:
        """A sink through which the product before this norm may carry out the norm's add and
        weighting itself, or None if this norm cannot finish such rows."""
        return None


    def forward(self, rt, x: torch.Tensor, delta, rows: torch.Tensor | None = None, unscaled_ok: bool = False):
        """x: the 32-bit residual stream [n, width], updated in place by `delta`
        (None, [n, width] or [splits, n, width]); returns the normalised rows in
        the runtime's element type.  rows: gather these rows only (x untouched).
        delta may be the `NormedRows` that a product made through this norm's sink (x is then
        up to date already); they are returned as they are if `unscaled_ok`, else scaled."""
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

    # A mixer or feed-forward that sets this takes `NormedRows` as h (it passes them to
    # `Runtime.linear` / `gated_linear` only) and a keyword `sink=` for its last product.
    takes_sinks = False

    def forward(self, rt, step, h: torch.Tensor, entry: int) -> torch.Tensor:
        """h: [T, width] normalised input.  entry: index of the schedule entry being run
        (names the cache line and the state through `step`).  Returns the update of the
        residual stream, [T, width] or [splits, T, width]."""
        raise NotImplementedError


class FeedForward(Part):
    takes_sinks = False  # as for Mixer

    def forward(self, rt, step, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    # a block that sets this takes `next_norm=` (the norm that will consume its pending update,
    # or None) and may hand that norm's sink to its last part
    takes_next_norm = False

    def forward(self, rt, step, x: torch.Tensor, pending, entry: int):
        """x: residual stream (in place); pending: an update not yet added to it (or the
        `NormedRows` of this block's first norm).  Returns (x, pending)."""
        raise NotImplementedError

    @property
    def first_norm(self):
        """The norm that takes this block's input, if the block before may feed it through a sink."""
        return None

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

"""The description of a whole model in terms of parts: what an architecture's
builder returns and what the engine turns into a running model."""
from __future__ import annotations

import dataclasses

from .base import PartSpec


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes ModelSpec.layers (a layer may be named
    by several entries: its weights are shared, each entry keeps a cache of its own).
    `reads_cache_of`: index of an earlier schedule entry whose keys and values this
    entry reads instead of keeping its own."""
    layer: int
    reads_cache_of: int | None = None


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab_size: int
    embedding: PartSpec
    position_encodings: dict[str, PartSpec]   # by name; mixers refer to them by name
    layers: tuple[PartSpec, ...]              # blocks
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int = 0                    # 0: no limit of the model's own
    stop_token_ids: tuple[int, ...] = ()

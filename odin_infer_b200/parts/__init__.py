"""Parts of a model: mixers, feed-forwards, norms, position encodings, blocks."""
from . import attention, block, embed_head, mlp, norm, position  # noqa: F401  (register the built-in parts)
from .base import (Block, Embedding, FeedForward, Head, Mixer, Norm, ParamSpec, Part, PartSpec, PositionEncoding,
                   build_part, register_part)
from .spec import ModelSpec, ScheduleEntry

__all__ = ["Block", "Embedding", "FeedForward", "Head", "Mixer", "ModelSpec", "Norm", "ParamSpec", "Part", "PartSpec",
           "PositionEncoding", "ScheduleEntry", "build_part", "register_part"]

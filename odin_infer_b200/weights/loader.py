"""Weights by tensor name from a model folder.

The model says which tensors it wants (`ParamSpec`s); the folder is checked
against that list as a whole, and ONE error names every missing tensor, every
unexpected one, and every wrong shape or element type.  The reference stops at
the first missing tensor and never checks a shape (infer/model.odin:82-97).

Element types: in the bfloat16 mode a tensor stored in bfloat16 or float16 is
kept as bfloat16 and a tensor stored in 32-bit stays 32-bit; integer tables
become int32.  In the float32 mode every floating tensor is widened to 32-bit.
"""
from __future__ import annotations

import torch

from ..parts.base import ParamSpec
from .safetensors_io import ModelFiles, SafetensorsError


class WeightError(ValueError):
    pass


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def check_folder(files: ModelFiles, specs: list[ParamSpec]) -> dict[str, str]:
    """Returns {wanted name: name in the files} or raises one WeightError."""
    have = set(files.names())
    wanted = {s.name for s in specs}
    alias_targets = {s.alias_of for s in specs if s.alias_of}
    missing, wrong = [], []
    source: dict[str, str] = {}
    for s in specs:
        if s.name in have:
            src = s.name
        elif s.alias_of is not None and (s.alias_of in have):
            src = s.alias_of
        else:
            missing.append(s.name + (f" (nor {s.alias_of})" if s.alias_of else ""))
            continue
        source[s.name] = src
        shape, dt = files.shape(src), files.dtype(src)
        if tuple(shape) != tuple(s.shape):
            wrong.append(f"{src}: shape {list(shape)}, expected {list(s.shape)}")
        elif s.is_integer and dt not in _INTS:
            wrong.append(f"{src}: element type {dt}, expected an integer type")
        elif not s.is_integer and dt not in _FLOATS:
            wrong.append(f"{src}: element type {dt}, expected float32, bfloat16 or float16")
    # a tied head may still be stored; it is then used as the head, never "unexpected"
    unexpected = sorted(have - wanted - alias_targets)
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: " + ", ".join(missing))
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: " + ", ".join(unexpected))
        if wrong:
            parts.append(f"{len(wrong)} wrong: " + "; ".join(wrong))
        raise WeightError("model folder does not match the model: " + " | ".join(parts))
    return source


def target_dtype(stored: torch.dtype, spec: ParamSpec, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.is_integer:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    return torch.float32 if stored == torch.float32 else torch.bfloat16


def load_weights(folder: str, specs: list[ParamSpec], compute_dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """Tensors by wanted name, on `device`; aliases share storage."""
    try:
        files = ModelFiles(folder)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    source = check_folder(files, specs)
    by_source: dict[str, torch.Tensor] = {}
    out: dict[str, torch.Tensor] = {}
    for s in specs:
        src = source[s.name]
        if src not in by_source:
            t = files.tensor(src)
            dt = target_dtype(t.dtype, s, compute_dtype)
            # move first, convert on the device: the host copy stays a view of the mapping
            by_source[src] = t.to(device=device).to(dtype=dt).contiguous()
        out[s.name] = by_source[src]
    return out

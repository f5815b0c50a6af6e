"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors straight in memory.

Matrices are N(0, 0.02), norm weights 1 + N(0, 0.1), integer tables zero.  Each
tensor has a generator of its own, seeded from (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or on their order.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config import ModelConfig, lookup_architecture
from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: ParamSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    if spec.is_integer:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    t = torch.empty(spec.shape, dtype=torch.float32, device=device)
    t.normal_(0.0, 1.0, generator=g)
    if spec.init == "norm":
        t.mul_(0.1).add_(1.0)
    elif spec.init == "matrix":
        t.mul_(0.02)
    else:
        raise ValueError(f"tensor '{spec.name}': unknown init '{spec.init}'")
    return t.to(dtype)


def model_param_specs(config: ModelConfig) -> list[ParamSpec]:
    """The tensors a model folder of this configuration holds (aliases left out)."""
    from ..engine.model import DecoderModel
    spec = lookup_architecture(config.architecture).build_spec(config)
    params = DecoderModel(spec).params()
    names = {p.name for p in params}
    return [p for p in params if not (p.alias_of is not None and p.alias_of in names)]


def write_random_model(folder: str, config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write config.json and model.safetensors; returns the folder."""
    os.makedirs(folder, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f, indent=1)
    params = model_param_specs(config)
    by_name = {p.name: p for p in params}
    write_safetensors(
        os.path.join(folder, "model.safetensors"),
        [(p.name, torch.int32 if p.is_integer else dtype, tuple(p.shape)) for p in params],
        lambda name: random_tensor(by_name[name], seed, dtype),
        metadata={"format": "pt", "seed": seed})
    return folder


def random_weights(specs: list[ParamSpec], seed: int, compute_dtype: torch.dtype, device,
                   stored_dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    """The same kind of tensors in memory, generated on `device` (values differ from a
    written folder's when the device differs, since generators are per device)."""
    out: dict[str, torch.Tensor] = {}
    names = {p.name for p in specs}
    for p in specs:
        if p.alias_of is not None and p.alias_of in names:
            continue
        t = random_tensor(p, seed, stored_dtype, device=device)
        out[p.name] = t if p.is_integer else t.to(torch.float32 if compute_dtype == torch.float32 else t.dtype)
    for p in specs:
        if p.name not in out:
            out[p.name] = out[p.alias_of]
    return out

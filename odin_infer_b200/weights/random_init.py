"""Random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed, or the same tensors straight in memory.

Matrices are N(0, 0.02), norm weights 1 + N(0, 0.1), integer tables zero.

The generator is counter-based: element i of the tensor called `name` under `seed` is a
function of (seed, name, i) alone, so a tensor's values do not depend on which other
tensors exist, on their order, on how the work is cut into chunks, or on whether the
host or the device computes them.  The device kernel (`odin_random_fill`) and the host
code below give the same bits; `Engine.random` weights can therefore be regenerated on
the host, tensor by tensor or row by row, without writing a folder.

    key   = mix64(mix64(seed) ^ fnv1a64(name))
    h1,h2 = mix64(key + 2 i), mix64(key + 2 i + 1)          (mix64: splitmix64's step)
    s     = sum of the eight 16-bit fields of h1 and h2      (0 .. 8 * 65535)
    value = mean + float32(s - 4 * 65535) * float32(std / sigma_s)

with sigma_s^2 = 8 (65536^2 - 1) / 12: a sum of eight uniforms (excess kurtosis -0.15
against the normal distribution's 0, bounded at 4.9 sigma), computed in integers so that
no library function's last bit can differ between host and device; the product and the
sum are single IEEE operations, and the rounding to bfloat16 is to nearest even.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch

from ..config import ModelConfig, lookup_architecture
from ..parts.base import ParamSpec
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1
_SIGMA_S = math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)
_CENTER = 4 * 65535
_INIT = {"matrix": (0.0, 0.02), "norm": (1.0, 0.1)}   # mean, standard deviation


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def _fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def stream_key(seed: int, name: str) -> int:
    """The 64-bit key of tensor `name` under `seed`."""
    return _mix64(_mix64(seed & _M64) ^ _fnv1a64(name))


def _mix64_np(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def host_values(key: int, start: int, count: int, mean: float, std: float) -> np.ndarray:
    """Elements [start, start + count) of the stream `key` as float32 (not yet rounded to a storage type)."""
    out = np.empty(count, dtype=np.float32)
    scale = np.float32(std / _SIGMA_S)
    chunk = 1 << 20
    with np.errstate(over="ignore"):
        for c0 in range(0, count, chunk):
            n = min(chunk, count - c0)
            i2 = (np.arange(start + c0, start + c0 + n, dtype=np.uint64) << np.uint64(1)) + np.uint64(key)
            s = np.zeros(n, dtype=np.uint64)
            for h in (_mix64_np(i2), _mix64_np(i2 + np.uint64(1))):
                for k in range(4):
                    s += (h >> np.uint64(16 * k)) & np.uint64(0xFFFF)
            c = (s.astype(np.int64) - _CENTER).astype(np.float32)
            out[c0:c0 + n] = np.float32(mean) + c * scale
    return out


def _to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even (the values here are finite)."""
    b = v.view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def host_tensor(name: str, shape, init: str, seed: int, dtype: torch.dtype, first_row: int = 0,
                n_rows: int | None = None) -> torch.Tensor:
    """Tensor `name` (or rows [first_row, first_row + n_rows) of it) computed on the host."""
    shape = tuple(shape)
    row = int(np.prod(shape[1:])) if len(shape) > 1 else 1
    rows = shape[0] if shape else 1
    n_rows = rows - first_row if n_rows is None else n_rows
    out_shape = (n_rows,) + shape[1:] if shape else ()
    mean, std = _INIT[init]
    v = host_values(stream_key(seed, name), first_row * row, n_rows * row, mean, std)
    if dtype == torch.bfloat16:
        t = torch.from_numpy(_to_bf16_bits(v).view(np.int16)).view(torch.bfloat16)
    else:
        t = torch.from_numpy(v).to(dtype)
    return t.reshape(out_shape)


def random_tensor(spec: ParamSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The tensor of `spec` under `seed`, stored as `dtype`; the same bits on the host and on a CUDA device."""
    if spec.is_integer:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    if spec.init not in _INIT:
        raise ValueError(f"tensor '{spec.name}': unknown init '{spec.init}'")
    if torch.device(device).type != "cuda":
        return host_tensor(spec.name, spec.shape, spec.init, seed, dtype)
    from ..csrc import ops
    mean, std = _INIT[spec.init]
    store = dtype if dtype in (torch.bfloat16, torch.float32) else torch.float32
    t = torch.empty(spec.shape, dtype=store, device=device)
    ops.random_fill(t, stream_key(seed, spec.name), mean, float(np.float32(std / _SIGMA_S)))
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
    """The same tensors in memory, generated on `device`: bit for bit those of a folder written
    with the same seed and `stored_dtype`."""
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

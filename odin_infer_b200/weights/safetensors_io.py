"""Reader and writer of the safetensors container, by tensor name.

A file is: 8 bytes little-endian header length, a JSON header
{name: {"dtype", "shape", "data_offsets": [begin, end]}}, then the raw data.
The reader maps the file and hands out tensors that alias the mapping (no copy
until the caller moves them to the device); the writer streams tensor by
tensor, so a model larger than host memory can be written.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Callable, Iterable

import torch

_TORCH_OF = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
             "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
             "BOOL": torch.bool}
_NAME_OF = {v: k for k, v in _TORCH_OF.items()}
_SIZE_OF = {"F32": 4, "BF16": 2, "F16": 2, "F64": 8, "I32": 4, "I64": 8, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: truncated (only {size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: truncated (header of {hlen} bytes does not fit in {size})")
        try:
            header = json.loads(self._f.read(hlen))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, dict] = header
        self._base = 8 + hlen
        for name, meta in header.items():
            dt, shape, (b, e) = meta.get("dtype"), meta.get("shape"), meta.get("data_offsets", (0, -1))
            if dt not in _SIZE_OF:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {dt!r}")
            n = 1
            for s in shape:
                n *= s
            if e - b != n * _SIZE_OF[dt]:
                raise SafetensorsError(f"{path}: tensor '{name}' has {e - b} bytes, its shape {shape} needs {n * _SIZE_OF[dt]}")
            if self._base + e > size:
                raise SafetensorsError(f"{path}: truncated (tensor '{name}' ends at byte {self._base + e} of {size})")
        # a private copy-on-write mapping: writable for torch.frombuffer, never written
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> list[str]:
        return list(self.entries)

    def dtype(self, name: str) -> torch.dtype:
        return _TORCH_OF[self.entries[name]["dtype"]]

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        meta = self.entries[name]
        b, e = meta["data_offsets"]
        dt = _TORCH_OF[meta["dtype"]]
        n = (e - b) // _SIZE_OF[meta["dtype"]]
        if n == 0:
            return torch.empty(tuple(meta["shape"]), dtype=dt)
        t = torch.frombuffer(self._map, dtype=dt, count=n, offset=self._base + b)
        return t.reshape(tuple(meta["shape"]))

    def close(self) -> None:
        # tensors handed out alias the mapping; it is closed when they are gone
        self._f.close()


class ModelFiles:
    """All safetensors files of a model folder, looked up by tensor name."""

    def __init__(self, folder: str):
        single = os.path.join(folder, "model.safetensors")
        if os.path.exists(single):
            paths = [single]
        else:
            paths = sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".safetensors"))
        if not paths:
            raise SafetensorsError(f"{folder}: no model.safetensors (nor any *.safetensors)")
        self.files = [SafetensorsFile(p) for p in paths]
        self.where: dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                if n in self.where:
                    raise SafetensorsError(f"tensor '{n}' is in both {self.where[n].path} and {f.path}")
                self.where[n] = f

    def names(self) -> list[str]:
        return list(self.where)

    def dtype(self, name: str) -> torch.dtype:
        return self.where[name].dtype(name)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.where[name].shape(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)


def write_safetensors(path: str, specs: Iterable[tuple[str, torch.dtype, tuple[int, ...]]],
                      make: Callable[[str], torch.Tensor], metadata: dict | None = None) -> None:
    """Write tensors one by one: `specs` gives (name, dtype, shape) in file order,
    `make(name)` the tensor when its turn comes."""
    specs = list(specs)
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, dt, shape in specs:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _SIZE_OF[_NAME_OF[dt]]
        header[name] = {"dtype": _NAME_OF[dt], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dt, shape in specs:
            t = make(name)
            if t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"tensor '{name}': made {t.dtype}{tuple(t.shape)}, promised {dt}{tuple(shape)}")
            t = t.contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() < (1 << 24)
                        else memoryview(t.view(torch.uint8).numpy()))
    os.replace(tmp, path)

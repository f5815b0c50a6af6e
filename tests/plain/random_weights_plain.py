"""Scalar restatement of the package's counter-based random weights, in Python integers.

The reference has no random-weights mode (infer/model.odin:82-97 only loads); the
generator is this package's own, so this file rests on its documented formula alone:

    key   = mix64(mix64(seed) ^ fnv1a64(name))
    h1,h2 = mix64(key + 2 i), mix64(key + 2 i + 1)
    s     = sum of the eight 16-bit fields of h1 and h2
    value = mean + float32(s - 4 * 65535) * float32(std / sqrt(8 (65536^2 - 1) / 12))

One element at a time, no numpy vector code, nothing imported from the package.
"""
from __future__ import annotations

import math
import struct

M = (1 << 64) - 1


def mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
    return z ^ (z >> 31)


def fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & M
    return h


def f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def element(seed: int, name: str, i: int, mean: float, std: float) -> float:
    """Element i (row-major) of tensor `name` under `seed`, as a float32 value."""
    key = mix64(mix64(seed & M) ^ fnv1a64(name))
    s = 0
    for h in (mix64((key + 2 * i) & M), mix64((key + 2 * i + 1) & M)):
        for k in range(4):
            s += (h >> (16 * k)) & 0xFFFF
    scale = f32(std / math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0))
    return f32(f32(mean) + f32(float(s - 4 * 65535) * scale))


def to_bf16(x: float) -> float:
    """Round a float32 value to the nearest bfloat16 (ties to even)."""
    (b,) = struct.unpack("<I", struct.pack("<f", x))
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return struct.unpack("<f", struct.pack("<I", b & 0xFFFFFFFF))[0]

"""Position encodings."""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_part


@register_part("position_encoding", "rope")
class RotaryEncoding(PositionEncoding):
    """Half-split rotary encoding: pairs (i, i + rotary_dim/2), frequency
    1 / theta^(i / (rotary_dim/2)), angle = position * frequency, both formed in
    32-bit as the reference does (infer/forward.odin:67-70); cos and sin of that
    angle are tabulated on the host, so every kernel reads the same values."""

    graph_safe = True

    def __init__(self, rotary_dim: int, theta: float):
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even, got {rotary_dim}")
        self.rotary_dim, self.theta = rotary_dim, float(theta)
        self.cos = self.sin = None

    def prepare(self, rt, n_positions: int) -> None:
        half = self.rotary_dim // 2
        i = np.arange(half, dtype=np.float32)
        freq = (np.float32(1.0) / np.power(np.float32(self.theta), i / np.float32(max(half, 1)))).astype(np.float32)
        pos = np.arange(max(n_positions, 1), dtype=np.float32)[:, None]
        ang = (pos * freq[None, :]).astype(np.float32).astype(np.float64)
        self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(rt.device).contiguous()
        self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(rt.device).contiguous()

    def rotation(self):
        return self.cos, self.sin, self.rotary_dim


@register_part("position_encoding", "none")
class NoEncoding(PositionEncoding):
    """No position information beyond the causal mask."""

    graph_safe = True

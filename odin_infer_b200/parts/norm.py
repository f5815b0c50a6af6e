"""RMSNorm with a plain weight, fused with the residual add that precedes it."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, ParamSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """o = w * (x / sqrt(mean(x^2) + eps)), in 32-bit (infer/ops.odin:7-19)."""

    graph_safe = True

    def __init__(self, width: int, eps: float, weight: str):
        self.width, self.eps, self.weight_name = width, float(eps), weight
        self.weight: torch.Tensor | None = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.width,), init="norm")]

    def bind(self, tensors, rt):
        self.weight = tensors[self.weight_name]

    def kernel_groups(self):
        return {"elementwise"}

    def forward(self, rt, x, delta, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.empty(n, self.width)
        ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        return out

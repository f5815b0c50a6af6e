"""Dense feed-forward parts."""
from __future__ import annotations

import torch

from .base import FeedForward, ParamSpec, register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """down( silu(gate(x)) * up(x) ), no bias (infer/forward.odin:125-135).  The gate
    and up matrices are fused into one at load time."""

    graph_safe = True

    def __init__(self, width: int, inner: int, names: dict):
        self.width, self.inner, self.names = width, inner, dict(names)
        self.w_gate_up = self.w_down = None

    def params(self):
        n = self.names
        return [ParamSpec(n["gate"], (self.inner, self.width)), ParamSpec(n["up"], (self.inner, self.width)),
                ParamSpec(n["down"], (self.width, self.inner))]

    def bind(self, tensors, rt):
        n = self.names
        g, u = tensors.pop(n["gate"]), tensors.pop(n["up"])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[n["down"]]

    def kernel_groups(self):
        return {"elementwise", "gemm_plain"}

    def notes(self, rt):
        if rt.dtype != torch.bfloat16:
            return []
        return [f"feed-forward: {what} = {k} is no multiple of 8: its matrix products run on CUDA cores "
                "(the tensor-core kernels read rows of whole 16 bytes)"
                for what, k in (("width", self.width), ("inner", self.inner)) if k % 8]

    takes_residual = True

    def forward(self, rt, step, h, residual=None):
        act = rt.gated_linear(h, self.w_gate_up, self.inner)
        return rt.linear(act, self.w_down, out_dtype=torch.float32, may_split=True, add_to=residual)

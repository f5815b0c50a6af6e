"""Token embedding and the output head."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Embedding, Head, ParamSpec, register_part


@register_part("embedding", "token_table")
class TokenEmbedding(Embedding):
    """x = E[token], no scaling (infer/forward.odin:43)."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str):
        self.vocab_size, self.width, self.weight_name = vocab_size, width, weight
        self.table = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width))]

    def bind(self, tensors, rt):
        self.table = tensors[self.weight_name]

    def kernel_groups(self):
        return {"elementwise"}

    def forward(self, rt, step):
        x = rt.empty(step.n_rows, self.width, dtype=torch.float32)
        ops.embed(self.table, step.tok_ids, x)
        return x


@register_part("head", "linear")
class LinearHead(Head):
    """logits = W h, 32-bit out; W is its own tensor or, when `tied_to` is given and
    the folder has no such tensor, the embedding table (infer/model.odin:150-158)."""

    graph_safe = True

    def __init__(self, vocab_size: int, width: int, weight: str, tied_to: str | None = None):
        self.vocab_size, self.width, self.weight_name, self.tied_to = vocab_size, width, weight, tied_to
        self.w = None

    def params(self):
        return [ParamSpec(self.weight_name, (self.vocab_size, self.width), alias_of=self.tied_to)]

    def bind(self, tensors, rt):
        self.w = tensors[self.weight_name]

    def kernel_groups(self):
        return {"gemm_plain"}

    def forward(self, rt, step, h):
        return rt.linear(h, self.w, out_dtype=torch.float32)

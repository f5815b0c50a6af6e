"""The runtime a part sees: the element type of activations, the device, scratch
tensors, and the choice between kernel variants for matrix products and
attention.  Parts never choose a kernel themselves."""
from __future__ import annotations

import torch

from ..csrc import ops


class Runtime:
    def __init__(self, device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype

    def kernel_groups(self) -> set[str]:
        """Kernel libraries the runtime itself may launch, beside those of the parts."""
        return set()

    def run(self, model, batch):
        """Run one step of `model`; returns the logits at the wanted rows."""
        return model.forward(self, batch)

    def empty(self, *shape, dtype: torch.dtype | None = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    # ---- matrix product: out[M, N] = a[M, K] @ w[N, K]^T -----------------
    def linear(self, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        out = self.empty(a.shape[0], w.shape[0], dtype=out_dtype or self.dtype)
        ops.gemm_plain(a, w, out)
        return out

    # ---- attention over the cache ---------------------------------------
    def attention(self, step, q, out, n_q, n_kv, head_dim, k_line, v_line, block_table, window) -> None:
        ops.attention_plain(q, out, n_q, n_kv, head_dim, k_line, v_line, step.tok_pos, step.tok_seq, block_table,
                            window)

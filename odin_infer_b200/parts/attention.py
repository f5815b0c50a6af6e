"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import torch

from ..cache import KVRequest
from ..csrc import ops
from .base import Mixer, ParamSpec, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Mixer):
    """q, k, v projections (no bias), optional per-head RMSNorm of q and k, rotation,
    causal attention of each query head h over kv head h // (n_q / n_kv), output
    projection.  Restates infer/forward.odin:53-117.

    window > 0 keeps only the last `window` keys visible.  kv_shared: this mixer has
    no k and v of its own and reads the cache line its schedule entry names.
    The three projection matrices are fused into one at load time.
    """

    graph_safe = True

    def __init__(self, width: int, n_q_heads: int, n_kv_heads: int, head_dim: int, names: dict,
                 position_encoding: str | None = None, qk_norm: bool = True, eps: float = 1e-6,
                 window: int = 0, kv_shared: bool = False):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} query heads are not a multiple of {n_kv_heads} kv heads")
        self.width, self.n_q, self.n_kv, self.hd = width, n_q_heads, n_kv_heads, head_dim
        self.names, self.pe_name = dict(names), position_encoding
        self.qk_norm, self.eps, self.window, self.kv_shared = qk_norm, float(eps), int(window), kv_shared
        self.pe = None          # set by the model from pe_name
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self._dummy = None

    def params(self):
        n = self.names
        out = [ParamSpec(n["q"], (self.n_q * self.hd, self.width))]
        if not self.kv_shared:
            out += [ParamSpec(n["k"], (self.n_kv * self.hd, self.width)),
                    ParamSpec(n["v"], (self.n_kv * self.hd, self.width))]
        out.append(ParamSpec(n["o"], (self.width, self.n_q * self.hd)))
        if self.qk_norm:
            out.append(ParamSpec(n["q_norm"], (self.hd,), init="norm"))
            if not self.kv_shared:
                out.append(ParamSpec(n["k_norm"], (self.hd,), init="norm"))
        return out

    def bind(self, tensors, rt):
        n = self.names
        if self.kv_shared:
            self.w_qkv = tensors[n["q"]]
        else:
            q, k, v = tensors.pop(n["q"]), tensors.pop(n["k"]), tensors.pop(n["v"])
            if not (q.dtype == k.dtype == v.dtype):
                q, k, v = (t.to(torch.float32) for t in (q, k, v))
            self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.qk_norm:
            self.q_norm = tensors[n["q_norm"]]
            self.k_norm = tensors[n["k_norm"]] if not self.kv_shared else self.q_norm
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        self._dummy = torch.zeros(1, 1, dtype=torch.float32, device=rt.device)

    def cache_request(self):
        return KVRequest(self.n_kv, self.hd, self.window)

    def kernel_groups(self):
        return {"head_prep", "attention_plain", "gemm_plain"}

    def notes(self, rt):
        import torch
        if rt.dtype != torch.bfloat16:
            return []
        out, hd, group = [], self.hd, self.n_q // self.n_kv
        rot = self.pe.rotation() if self.pe is not None else None
        if not ops.attention_prefill_supported(hd):
            out.append(f"attention: head_dim {hd} is not 64 or 128: prompts run the CUDA-core attention kernel "
                       "(one warp per token and head), far slower than the tensor-core one")
        if not ops.attention_decode_supported(hd):
            out.append(f"attention: head_dim {hd} is no power of two from 16 to 256: decoding runs the CUDA-core "
                       "attention kernel without key splits")
        elif hd not in (64, 128) or group > 16:
            out.append(f"attention: head_dim {hd} with {group} query heads per kv head: decoding runs the CUDA-core "
                       "split-key kernel (the tensor-core one takes head_dim 64 or 128 and up to 16 query heads per kv head)")
        elif rot is not None and rot[2] != hd:
            out.append(f"attention: rotary_dim {rot[2]} < head_dim {hd}: head preparation runs as a kernel of its own "
                       "when decoding")
        for what, k in (("width", self.width), ("n_q_heads * head_dim", self.n_q * hd)):
            if k % 8:
                out.append(f"attention: {what} = {k} is no multiple of 8: its matrix products run on CUDA cores "
                           "(the tensor-core kernels read rows of whole 16 bytes)")
        return out

    takes_residual = True

    def forward(self, rt, step, h, entry, residual=None):
        T = h.shape[0]
        qkv = rt.linear(h, self.w_qkv, may_split=True, beside_attention=True)
        k_line, v_line, block_table = step.kv(entry)
        rot = self.pe.rotation() if self.pe is not None else None
        cos, sin, rot_dim = rot if rot is not None else (self._dummy, self._dummy, 0)
        writes = step.writes_cache(entry) and not self.kv_shared
        o = rt.empty(T, self.n_q * self.hd)
        # decoding: the attention kernel may prepare its heads itself
        if not self.kv_shared and rt.attention_with_head_prep(
                step, qkv, o, self.n_q, self.n_kv, self.hd, self.q_norm if self.qk_norm else None,
                self.k_norm if self.qk_norm else None, self.eps, cos, sin, rot_dim, k_line, v_line, block_table,
                self.window, writes):
            return rt.linear(o, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True, add_to=residual)
        # a product of few tokens may come back as partial sums: they are added here
        q_out = rt.empty(T, self.n_q * self.hd) if qkv.dim() == 3 else None
        q = ops.head_prep(qkv, self.n_q, 0 if self.kv_shared else self.n_kv, self.hd,
                          self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None, self.eps,
                          cos, sin, rot_dim, step.tok_pos, step.tok_seq, block_table, k_line, v_line,
                          write_kv=writes, q_out=q_out)
        rt.attention(step, q, o, self.n_q, self.n_kv, self.hd, k_line, v_line, block_table, self.window)
        return rt.linear(o, self.w_o, out_dtype=torch.float32, may_split=True, beside_attention=True, add_to=residual)

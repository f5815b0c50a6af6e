"""A second, independently structured restatement of the reference's forward pass, in numpy
float64: one token at a time with key and value arrays per layer, exactly the shape of
`forward(transformer, token, pos)` (infer/forward.odin:17-146), where qwen3_plain.py works on
whole sequences with matrix products.  The two share no arithmetic; a test demands that they
agree to float64 rounding, so the oracle does not rest on one reading of the reference.

Like qwen3_plain.py it rests on the reference's formulas (cited by line): the reference is an
Odin program and this image has no Odin compiler.
"""
from __future__ import annotations

import math

import numpy as np


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """infer/ops.odin:7-19: ss = sum x^2; ss /= n; ss += eps; ss = 1/sqrt(ss); o = w * (ss * x)."""
    ss = 0.0
    for v in x:
        ss += v * v
    ss /= len(x)
    ss += eps
    ss = 1.0 / math.sqrt(ss)
    return w * (ss * x)


def softmax(a: np.ndarray) -> np.ndarray:
    """infer/ops.odin:21-37: subtract the maximum, exponentiate, divide by the sum."""
    m = a[0]
    for v in a[1:]:
        if v > m:
            m = v
    e = np.array([math.exp(v - m) for v in a])
    total = 0.0
    for v in e:
        total += v
    return e / total


def matvec(w: np.ndarray, x: np.ndarray) -> np.ndarray:
    """infer/matmul.odin:63-70: out[row] = sum_j w[row, j] x[j]."""
    return np.array([np.dot(w[r], x) for r in range(w.shape[0])])


class Stepwise:
    """The reference's Transformer with its run state (infer/model.odin:12-24, :36-60)."""

    def __init__(self, cfg: dict, weights: dict, seq_len: int):
        self.dim = cfg["hidden_size"]
        self.hidden_dim = cfg["intermediate_size"]
        self.n_layers = cfg["num_hidden_layers"]
        self.n_heads = cfg["num_attention_heads"]
        self.n_kv_heads = cfg.get("num_key_value_heads", self.n_heads)
        self.head_dim = cfg.get("head_dim", self.dim // self.n_heads)
        self.rope_freq = np.float32(cfg.get("rope_theta", 1e6))     # infer/model.odin:125-129
        self.eps = cfg.get("rms_norm_eps", 1e-6)                    # infer/model.odin:130-134
        self.seq_len = seq_len
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        kv_dim = self.n_kv_heads * self.head_dim
        self.key_cache = np.zeros((self.n_layers, seq_len, kv_dim))
        self.value_cache = np.zeros((self.n_layers, seq_len, kv_dim))

    def forward(self, token: int, pos: int) -> np.ndarray:
        """Logits [vocab] of `token` at `pos`, given the cache that positions < pos left."""
        assert 0 <= pos < self.seq_len                               # infer/forward.odin:22-25
        w, hd, half = self.w, self.head_dim, self.head_dim // 2
        kv_mul = self.n_heads // self.n_kv_heads
        x = w["model.embed_tokens.weight"][token].copy()             # :43
        for l in range(self.n_layers):
            p = f"model.layers.{l}."
            xb = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)                     # :51
            q = matvec(w[p + "self_attn.q_proj.weight"], xb)                               # :53
            k = matvec(w[p + "self_attn.k_proj.weight"], xb)                               # :54
            v = matvec(w[p + "self_attn.v_proj.weight"], xb)                               # :55
            for h in range(self.n_heads):                                                  # :58-86
                qh = rmsnorm(q[h * hd:(h + 1) * hd], w[p + "self_attn.q_norm.weight"], self.eps)
                kh = None
                if h < self.n_kv_heads:
                    kh = rmsnorm(k[h * hd:(h + 1) * hd], w[p + "self_attn.k_norm.weight"], self.eps)
                for i in range(half):
                    # frequency and angle are formed in 32-bit (:68-70), cos and sin taken of that angle
                    freq = np.float32(1.0) / np.power(self.rope_freq, np.float32(i) / np.float32(half), dtype=np.float32)
                    ang = float(np.float32(pos) * freq)
                    fcr, fci = math.cos(ang), math.sin(ang)
                    xq, yq = qh[i], qh[i + half]
                    qh[i], qh[i + half] = xq * fcr - yq * fci, xq * fci + yq * fcr
                    if kh is not None:
                        xk, yk = kh[i], kh[i + half]
                        kh[i], kh[i + half] = xk * fcr - yk * fci, xk * fci + yk * fcr
                q[h * hd:(h + 1) * hd] = qh
                if kh is not None:
                    k[h * hd:(h + 1) * hd] = kh
            self.key_cache[l, pos] = k
            self.value_cache[l, pos] = v
            xb3 = np.zeros(self.n_heads * hd)
            for h in range(self.n_heads):                                                  # :89-115
                qh = q[h * hd:(h + 1) * hd]
                off = (h // kv_mul) * hd
                att = np.empty(pos + 1)
                for t in range(pos + 1):
                    att[t] = np.dot(qh, self.key_cache[l, t, off:off + hd]) / math.sqrt(hd)
                att = softmax(att)
                acc = np.zeros(hd)
                for t in range(pos + 1):
                    acc += att[t] * self.value_cache[l, t, off:off + hd]
                xb3[h * hd:(h + 1) * hd] = acc
            x = x + matvec(w[p + "self_attn.o_proj.weight"], xb3)                          # :117-121
            xb = rmsnorm(x, w[p + "post_attention_layernorm.weight"], self.eps)            # :123
            hb = matvec(w[p + "mlp.gate_proj.weight"], xb)                                 # :125
            hb2 = matvec(w[p + "mlp.up_proj.weight"], xb)                                  # :126
            for i in range(self.hidden_dim):                                               # :128-133
                val = hb[i]
                val *= 1.0 / (1.0 + math.exp(-val))
                val *= hb2[i]
                hb2[i] = val
            x = x + matvec(w[p + "mlp.down_proj.weight"], hb2)                             # :135-139
        x = rmsnorm(x, w["model.norm.weight"], self.eps)                                   # :142
        head = w.get("lm_head.weight", w["model.embed_tokens.weight"])                     # infer/model.odin:150-158
        return matvec(head, x)                                                             # :143


def logits_token_by_token(cfg: dict, weights: dict, tokens) -> np.ndarray:
    """[len(tokens), vocab]: the reference's generation loop without sampling (teacher-forced)."""
    m = Stepwise(cfg, weights, len(tokens))
    return np.stack([m.forward(int(t), pos) for pos, t in enumerate(tokens)])

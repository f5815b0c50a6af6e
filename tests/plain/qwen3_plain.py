"""Plain, slow implementation of the Qwen3 dense decoder: the oracle of the tests.

Whole sequences, no cache, one function per part, float32 (or float64) on the
CPU.  It shares no code with the product package: it has its own reader of
config.json and of the safetensors container and its own arithmetic.

It rests on the formulas of the reference's CPU forward pass (the reference is
written in Odin, for which this image has no compiler, so its model code could
not be imported or compiled for a cross-check; every function below cites the
lines it restates, by the file's path within the reference project).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# --------------------------------------------------------------------------
# model folder reader (own code: a safetensors file is an 8-byte little-endian
# header length, a JSON header {name: {dtype, shape, data_offsets}}, raw data)
# --------------------------------------------------------------------------
_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2),
              "I32": (np.int32, 4), "I64": (np.int64, 8), "F64": (np.float64, 8)}


def read_model_folder(folder: str, dtype=torch.float32):
    """Return (config dict, {tensor name: torch tensor of `dtype`})."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        base = 8 + hlen
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            npdt, _ = _ST_DTYPES[meta["dtype"]]
            b, e = meta["data_offsets"]
            f.seek(base + b)
            raw = np.frombuffer(f.read(e - b), dtype=npdt).reshape(meta["shape"])
            if meta["dtype"] == "BF16":
                # a bfloat16 is the upper half of a float32
                t = torch.from_numpy((raw.astype(np.uint32) << 16).view(np.float32).copy())
            else:
                t = torch.from_numpy(raw.copy())
            tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, tensors


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens) -> torch.Tensor:
    """x = E[token, :], no scaling.  infer/forward.odin:43, :12-15."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2 / size + eps; o = w * ((1/sqrt(ss)) * x).  infer/ops.odin:7-19."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    ss = ss + eps
    r = 1.0 / torch.sqrt(ss)
    return weight * (r * x)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[row] = sum_j W[row, j] x[j], no bias.  infer/matmul.odin:63-70, :77."""
    return x @ w.t()


def rope_tables(n_pos: int, head_dim: int, theta: float, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """freq_i = 1 / theta^(i / (hd/2)); angle = pos * freq.  infer/forward.odin:67-70.

    The reference forms the frequency and the angle in 32-bit; so does this
    (float32 products), and then takes cos and sin of that angle.
    """
    half = head_dim // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), i / np.float32(half))).astype(np.float32)
    pos = np.arange(n_pos, dtype=np.float32)[:, None]
    ang = (pos * freq[None, :]).astype(np.float32).astype(np.float64)
    return (torch.from_numpy(np.cos(ang)).to(dtype), torch.from_numpy(np.sin(ang)).to(dtype))


def rope(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split pairs (i, i + hd/2): (x, y) -> (x c - y s, x s + y c).

    v: [T, heads, hd]; cos, sin: [T, hd/2].  infer/forward.odin:72-75.
    """
    half = v.shape[-1] // 2
    x, y = v[..., :half], v[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x * c - y * s, x * s + y * c], dim=-1)


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    """m = max; e = exp(s - m); e / sum e.  infer/ops.odin:21-37."""
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """q: [T, Hq, hd]; k, v: [T, Hkv, hd] -> [T, Hq*hd].

    Query head h reads kv head h // (Hq/Hkv); score_t = q.k_t / sqrt(hd) for
    t <= pos (the causal mask is the loop bound); softmax; out = sum_t p_t v_t.
    infer/forward.odin:88-115.  `window` > 0 keeps only the last `window` keys
    (t > pos - window); the reference has no window, 0 means all keys.
    """
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    out = torch.zeros(T, Hq, hd, dtype=q.dtype)
    t_idx = torch.arange(T)
    allowed = t_idx[None, :] <= t_idx[:, None]
    if window > 0:
        allowed &= t_idx[None, :] > (t_idx[:, None] - window)
    for h in range(Hq):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].t()) / math.sqrt(hd)
        s = s.masked_fill(~allowed, float("-inf"))
        p = softmax_rows(s)
        out[:, h, :] = p @ v[:, kh, :]
    return out.reshape(T, Hq * hd)


def swiglu_mlp(x: torch.Tensor, w_gate, w_up, w_down) -> torch.Tensor:
    """h = gate * (1/(1+exp(-gate))) * up; out = W2 h.  infer/forward.odin:125-135."""
    g = linear(x, w_gate)
    u = linear(x, w_up)
    h = g * (1.0 / (1.0 + torch.exp(-g))) * u
    return linear(h, w_down)


def attention_block(x, w, prefix, cfg, cos, sin) -> torch.Tensor:
    """q,k,v projections, per-head q/k RMSNorm, RoPE, attention, output
    projection.  infer/forward.odin:53-117."""
    T = x.shape[0]
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[prefix + "q_proj.weight"]).reshape(T, Hq, hd)
    k = linear(x, w[prefix + "k_proj.weight"]).reshape(T, Hkv, hd)
    v = linear(x, w[prefix + "v_proj.weight"]).reshape(T, Hkv, hd)
    q = rmsnorm(q, w[prefix + "q_norm.weight"], eps)
    k = rmsnorm(k, w[prefix + "k_norm.weight"], eps)
    q = rope(q, cos, sin)
    k = rope(k, cos, sin)
    o = causal_attention(q, k, v)
    return linear(o, w[prefix + "o_proj.weight"])


def decoder_layer(x, w, l, cfg, cos, sin) -> torch.Tensor:
    """x + Attn(RMSNorm(x)), then x + MLP(RMSNorm(x)).  infer/forward.odin:51, :117-139."""
    p = f"model.layers.{l}."
    eps = cfg["rms_norm_eps"]
    h = rmsnorm(x, w[p + "input_layernorm.weight"], eps)
    x = x + attention_block(h, w, p + "self_attn.", cfg, cos, sin)
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                       w[p + "mlp.down_proj.weight"])
    return x


def normalise_config(cfg: dict) -> dict:
    cfg = dict(cfg)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    cfg.setdefault("rope_theta", 1e6)       # infer/model.odin:125-129
    cfg.setdefault("rms_norm_eps", 1e-6)    # infer/model.odin:130-134
    cfg.setdefault("tie_word_embeddings", False)
    return cfg


def forward_whole(cfg: dict, w: dict, tokens, positions=None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (or [len(positions), V] at the
    given ones: the final norm and the head act on single rows).  infer/forward.odin:17-146.

    The head is lm_head.weight if the folder has it, else the embedding table
    (infer/model.odin:150-158).
    """
    cfg = normalise_config(cfg)
    dtype = w["model.embed_tokens.weight"].dtype
    T = len(tokens)
    cos, sin = rope_tables(T, cfg["head_dim"], cfg["rope_theta"], dtype)
    x = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, l, cfg, cos, sin)
    if positions is not None:
        x = x[torch.as_tensor(list(positions), dtype=torch.long)]
    x = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return linear(x, head)


# --------------------------------------------------------------------------
# sampler (host restatement of sampler/sampler.odin)
# --------------------------------------------------------------------------
def argmax_first(logits) -> int:
    """First maximum wins (strict >).  sampler/sampler.odin:79-89."""
    best, best_i = logits[0], 0
    for i in range(1, len(logits)):
        if logits[i] > best:
            best, best_i = logits[i], i
    return best_i


def temperature_probs(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """logits / T, then softmax.  sampler/sampler.odin:179-182."""
    return softmax_rows((logits / temperature)[None, :])[0]


def sample_mult(probs, coin: float) -> int:
    """Walk the CDF in index order; first i with coin < cdf.  sampler/sampler.odin:91-100."""
    cdf = 0.0
    for i, p in enumerate(probs):
        cdf += float(p)
        if coin < cdf:
            return i
    return len(probs) - 1


def top_p_keep(probs: torch.Tensor, topp: float) -> set:
    """The set of tokens that top-p keeps: sort descending, keep until the
    cumulative probability first exceeds topp.  sampler/sampler.odin:106-128."""
    n = len(probs)
    cutoff = (1.0 - topp) / (n - 1)
    cand = [(float(p), i) for i, p in enumerate(probs) if float(p) >= cutoff]
    cand.sort(key=lambda t: -t[0])
    cum, keep = 0.0, set()
    for p, i in cand:
        cum += p
        keep.add(i)
        if cum > topp:
            break
    return keep


def sample_topp(probs, topp: float, coin: float):
    """The reference's top-p draw: candidates with p >= (1 - topp) / (n - 1), sorted by falling
    probability, cut after the first whose cumulative sum exceeds topp, the coin scaled by that
    sum, and a walk of the sorted list.  sampler/sampler.odin:106-139.

    Returns (token, margin): margin is how far (in probability) the scaled coin lies from the
    nearer end of the chosen token's interval; a draw with a tiny margin may go to the neighbour
    under another rounding of the sums."""
    n = len(probs)
    cutoff = (1.0 - topp) / (n - 1)
    cand = [(float(p), i) for i, p in enumerate(probs) if float(p) >= cutoff]
    cand.sort(key=lambda t: -t[0])           # stable: equal probabilities stay in index order
    cumulative, last_idx = 0.0, len(cand) - 1
    for j, (p, _) in enumerate(cand):
        cumulative += p
        if cumulative > topp:
            last_idx = j
            break
    r = coin * cumulative
    cdf = 0.0
    for j in range(last_idx + 1):
        before = cdf
        cdf += cand[j][0]
        if r < cdf:
            return cand[j][1], (cdf - r) if j == 0 else min(r - before, cdf - r)
    return cand[last_idx][1], 0.0


def repetition_penalty(logits: torch.Tensor, recent, penalty: float) -> torch.Tensor:
    """Each distinct recent token: divide a positive logit, multiply a negative
    one.  sampler/sampler.odin:143-160."""
    out = logits.clone()
    for t in set(int(t) for t in recent):
        if 0 <= t < len(out):
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out

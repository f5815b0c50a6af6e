"""Configuration of the Qwen3 dense decoder.

The reference reads the same quantities from GGUF metadata into its `Config`
(infer/model.odin:12-24, :99-139: embedding_length, feed_forward_length,
block_count, head_count, head_count_kv, context_length, key_length,
rope.freq_base default 1e6, layer_norm_rms_epsilon default 1e-6).  Here they
come from the config.json keys of a model folder.  The reference has no
attention bias, no sliding window, SiLU only, full rotary: a config.json that
asks for anything else is refused.
"""
from __future__ import annotations

import dataclasses

from .base import KeyReader, ModelConfig


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    vocab_size: int = 0
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 0     # 0: not given; the engine's context cap rules alone
    eos_token_id: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "Qwen3Config":
        r = KeyReader(raw, where)
        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        d = r.get("hidden_size", int)
        inter = r.get("intermediate_size", int)
        layers = r.get("num_hidden_layers", int)
        hq = r.get("num_attention_heads", int)
        hkv = r.get("num_key_value_heads", int, hq)
        hd = r.get("head_dim", int, (d // hq) if hq else 0)
        vocab = r.get("vocab_size", int)
        theta = r.get("rope_theta", float, 1e6)
        eps = r.get("rms_norm_eps", float, 1e-6)
        tie = r.get("tie_word_embeddings", bool, False)
        max_pos = r.get("max_position_embeddings", int, 0)
        eos = raw.get("eos_token_id", None)
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            r.problems.append(f"key 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
            eos_ids = ()
        for key, val in (("hidden_size", d), ("intermediate_size", inter), ("num_hidden_layers", layers),
                         ("num_attention_heads", hq), ("num_key_value_heads", hkv), ("head_dim", hd),
                         ("vocab_size", vocab)):
            r.require(val > 0 or f"missing key '{key}'" in r.problems, f"key '{key}' must be positive, got {val}")
        if hq > 0 and hkv > 0:
            r.require(hq % hkv == 0, f"num_attention_heads ({hq}) is not a multiple of num_key_value_heads ({hkv})")
        r.require(hd % 2 == 0, f"head_dim ({hd}) must be even for the half-split rotation")
        r.require(theta > 0, f"rope_theta must be positive, got {theta}")
        r.require(eps > 0, f"rms_norm_eps must be positive, got {eps}")
        r.require(not raw.get("attention_bias", False), "attention_bias is not supported (this architecture has no bias tensors)")
        r.require(raw.get("hidden_act", "silu") == "silu", f"hidden_act must be 'silu', got {raw.get('hidden_act')!r}")
        if raw.get("use_sliding_window", False) and raw.get("sliding_window") is not None:
            r.problems.append("sliding-window attention is not part of this architecture")
        r.require(raw.get("rope_scaling") in (None, {}), "rope_scaling is not supported")
        r.finish()
        return cls(architecture=str(archs[0]), hidden_size=d, intermediate_size=inter, num_hidden_layers=layers,
                   num_attention_heads=hq, num_key_value_heads=hkv, head_dim=hd, vocab_size=vocab,
                   rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tie, max_position_embeddings=max_pos,
                   eos_token_id=eos_ids, torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture], "model_type": "qwen3", "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "vocab_size": self.vocab_size, "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps, "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu", "attention_bias": False, "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id) if len(self.eos_token_id) > 1 else self.eos_token_id[0]
        return out

    def stop_token_ids(self) -> tuple[int, ...]:
        return self.eos_token_id

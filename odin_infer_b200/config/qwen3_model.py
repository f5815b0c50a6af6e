"""The Qwen3 dense decoder written out in parts.

Every layer: pre-norm block of RMSNorm, grouped-query attention with per-head
q/k RMSNorm and full rotary encoding, RMSNorm, SwiGLU; then a final RMSNorm and
a head that is its own tensor or the embedding table.  The tensor names are the
ones of a "config.json plus safetensors" model folder; the reference keeps the
same roles under GGUF names (infer/model.odin:146-177: token_embd, attn_norm,
attn_q/k/v, attn_q_norm, attn_k_norm, attn_output, ffn_norm, ffn_gate/up/down,
output_norm, output).
"""
from __future__ import annotations

from ..parts.base import PartSpec
from ..parts.spec import ModelSpec, ScheduleEntry
from .qwen3 import Qwen3Config
from .registry import register_architecture


def build_qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        mixer = PartSpec("gqa_attention", dict(
            width=cfg.hidden_size, n_q_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, position_encoding="rope", qk_norm=True, eps=cfg.rms_norm_eps, window=0,
            names={"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                   "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
                   "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"}))
        ffn = PartSpec("swiglu", dict(
            width=cfg.hidden_size, inner=cfg.intermediate_size,
            names={"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                   "down": p + "mlp.down_proj.weight"}))
        norm1 = PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps, weight=p + "input_layernorm.weight"))
        norm2 = PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                         weight=p + "post_attention_layernorm.weight"))
        layers.append(PartSpec("prenorm", dict(mixer=mixer, feed_forward=ffn, norm_mixer=norm1, norm_feed_forward=norm2)))
    return ModelSpec(
        width=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab_size, width=cfg.hidden_size,
                                               weight="model.embed_tokens.weight")),
        position_encodings={"rope": PartSpec("rope", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta))},
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l) for l in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps, weight="model.norm.weight")),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab_size, width=cfg.hidden_size, weight="lm_head.weight",
                                     tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None)),
        max_positions=cfg.max_position_embeddings,
        stop_token_ids=cfg.stop_token_ids(),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec)

"""Tiny configurations and helpers shared by the tests.

TINY_A and TINY_B differ in every size and option of the architecture: layers,
width, heads and groups, head size, q width equal to / different from the
width, intermediate size, vocabulary (neither a power of two in B), rope theta,
norm eps, tied / untied head.  TINY_C has a head size of 48 and 5 query heads on
one kv head.
"""
from __future__ import annotations

import os

import numpy as np
import torch

TINY_A = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=224, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=384, rope_theta=1e6,
              rms_norm_eps=1e-5, tie_word_embeddings=False, eos_token_id=[7, 9])
TINY_C = dict(architectures=["Qwen3ForCausalLM"], hidden_size=72, intermediate_size=200, num_hidden_layers=1,
              num_attention_heads=5, num_key_value_heads=1, head_dim=48, vocab_size=301, rope_theta=5e5,
              rms_norm_eps=1e-6, tie_word_embeddings=False)

# head sizes 64 and 128: the ones the tensor-core attention kernels take
TINY_D = dict(architectures=["Qwen3ForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=512, rope_theta=1e6,
              rms_norm_eps=1e-6, tie_word_embeddings=True)
TINY_E = dict(architectures=["Qwen3ForCausalLM"], hidden_size=192, intermediate_size=320, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=1, head_dim=128, vocab_size=1000, rope_theta=1e4,
              rms_norm_eps=1e-5, tie_word_embeddings=False)

TINIES = {"A": (TINY_A, 0), "B": (TINY_B, 2), "C": (TINY_C, 8), "D": (TINY_D, 11), "E": (TINY_E, 12)}  # config, weight seed


def make_folder(tmp_path, raw: dict, seed: int, dtype=torch.bfloat16) -> str:
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"model_{seed}_{raw['hidden_size']}")
    return write_random_model(folder, config_from_dict(raw), seed, dtype)


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def plain_logits(folder: str, tokens, dtype=torch.float64) -> np.ndarray:
    """[len(tokens), vocab] from the plain implementation."""
    from tests.plain import qwen3_plain
    cfg, w = qwen3_plain.read_model_folder(folder, dtype)
    return qwen3_plain.forward_whole(cfg, w, tokens).to(torch.float64).numpy()


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Largest absolute difference, relative to the largest reference magnitude."""
    return float(np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


# Tolerances on rel_err, fixed before the engine existed.  float32: sums of a few
# hundred terms, a few layers.  bfloat16: 8 bits of mantissa (2^-9 per rounding) on
# activations and cache, accumulated over the layers of the tiny models.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}

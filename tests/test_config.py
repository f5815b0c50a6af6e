"""Configuration and registry (no GPU)."""
import json

import pytest

from odin_infer_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures, load_config,
                                    lookup_architecture)
from tests import tiny


def test_reads_every_key_and_defaults():
    c = config_from_dict(tiny.TINY_B)
    assert isinstance(c, Qwen3Config)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 224, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 2, 32)
    assert c.vocab_size == 384 and c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5
    assert c.tie_word_embeddings is False and c.eos_token_id == (7, 9) and c.stop_token_ids() == (7, 9)
    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2,
               num_attention_heads=4, vocab_size=100)
    d = config_from_dict(raw)
    # defaults as the reference's loader has them (infer/model.odin:125-134)
    assert d.num_key_value_heads == 4 and d.head_dim == 16 and d.rope_theta == 1e6 and d.rms_norm_eps == 1e-6
    assert d.tie_word_embeddings is False and d.eos_token_id == ()


def test_round_trip_through_config_json(tmp_path):
    c = config_from_dict(tiny.TINY_A)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c


def test_all_problems_in_one_error():
    raw = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=6,
               num_key_value_heads=4, head_dim=15, vocab_size=100, attention_bias=True, hidden_act="gelu")
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    msg = str(e.value)
    for piece in ("intermediate_size", "not a multiple", "head_dim", "attention_bias", "hidden_act"):
        assert piece in msg, (piece, msg)


def test_refuses_what_the_architecture_does_not_have():
    with pytest.raises(ConfigError, match="sliding-window"):
        config_from_dict(dict(tiny.TINY_A, use_sliding_window=True, sliding_window=128))
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(dict(tiny.TINY_A, rope_scaling={"type": "yarn", "factor": 4}))
    assert config_from_dict(dict(tiny.TINY_A, use_sliding_window=False, sliding_window=None)).hidden_size == 64


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    assert lookup_architecture("Qwen3ForCausalLM").config_class is Qwen3Config
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'"):
        config_from_dict(dict(tiny.TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 64})


def test_spec_has_no_size_of_its_own():
    """Everything in the model description comes from the configuration."""
    for raw in (tiny.TINY_A, tiny.TINY_B, tiny.TINY_C):
        c = config_from_dict(raw)
        spec = lookup_architecture(c.architecture).build_spec(c)
        assert len(spec.layers) == raw["num_hidden_layers"] == len(spec.schedule)
        m = spec.layers[0].args["mixer"].args
        assert (m["n_q_heads"], m["n_kv_heads"], m["head_dim"]) == (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert spec.layers[0].args["feed_forward"].args["inner"] == raw["intermediate_size"]
        assert spec.position_encodings["rope"].args == dict(rotary_dim=raw["head_dim"], theta=raw["rope_theta"])
        assert spec.final_norm.args["eps"] == raw["rms_norm_eps"]
        assert (spec.head.args["tied_to"] is not None) == raw["tie_word_embeddings"]

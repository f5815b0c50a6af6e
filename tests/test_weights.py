"""Weights by name, the one error, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from odin_infer_b200.config import config_from_dict
from odin_infer_b200.weights import (ModelFiles, SafetensorsError, WeightError, load_weights, model_param_specs,
                                     write_safetensors)
from tests import tiny


def specs_of(raw):
    from odin_infer_b200.config import lookup_architecture
    from odin_infer_b200.engine.model import DecoderModel
    c = config_from_dict(raw)
    return DecoderModel(lookup_architecture(c.architecture).build_spec(c)).params()


def rewrite(folder, change):
    """Rewrite model.safetensors after `change(dict of tensors)`."""
    files = ModelFiles(folder)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    change(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], lambda n: tensors[n])


def test_random_folder_loads_and_is_deterministic(tmp_path):
    a = tiny.make_folder(tmp_path / "a", tiny.TINY_B, 2)
    b = tiny.make_folder(tmp_path / "b", tiny.TINY_B, 2)
    c = tiny.make_folder(tmp_path / "c", tiny.TINY_B, 3)
    fa, fb, fc = ModelFiles(a), ModelFiles(b), ModelFiles(c)
    assert sorted(fa.names()) == sorted(p.name for p in model_param_specs(config_from_dict(tiny.TINY_B)))
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert not torch.equal(fa.tensor("lm_head.weight"), fc.tensor("lm_head.weight"))
    w = fa.tensor("model.layers.0.mlp.up_proj.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = fa.tensor("model.norm.weight").float()
    assert abs(n.mean().item() - 1) < 0.05
    assert json.load(open(os.path.join(a, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]


def test_dtypes_kept(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, 0)
    rewrite(folder, lambda t: t.update({"model.norm.weight": t["model.norm.weight"].float()}))
    specs = specs_of(tiny.TINY_A)
    bf = load_weights(folder, specs, torch.bfloat16, "cpu")
    assert bf["model.norm.weight"].dtype == torch.float32          # stored in 32-bit: stays so
    assert bf["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    f32 = load_weights(folder, specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["model.embed_tokens.weight"], bf["model.embed_tokens.weight"].float())


def test_tied_head_aliases_the_table(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, 0)
    w = load_weights(folder, specs_of(tiny.TINY_A), torch.bfloat16, "cpu")
    assert w["lm_head.weight"].data_ptr() == w["model.embed_tokens.weight"].data_ptr()
    # an untied configuration with the head missing is an error that names it
    os.remove(os.path.join(folder, "config.json"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(folder, specs_of(dict(tiny.TINY_A, tie_word_embeddings=False)), torch.bfloat16, "cpu")


def test_one_error_lists_everything(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_B, 2)

    def change(t):
        del t["model.layers.1.self_attn.k_norm.weight"]
        del t["model.layers.2.mlp.down_proj.weight"]
        t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192)
        t["extra.tensor"] = torch.zeros(3)
        t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(224, 95, dtype=torch.bfloat16)
        t["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    rewrite(folder, change)
    with pytest.raises(WeightError) as e:
        load_weights(folder, specs_of(tiny.TINY_B), torch.bfloat16, "cpu")
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.self_attn.k_norm.weight" in msg and "model.layers.2.mlp.down_proj.weight" in msg
    assert "2 unexpected" in msg and "extra.tensor" in msg and "model.layers.0.self_attn.q_proj.bias" in msg
    assert "2 wrong" in msg and "[224, 95], expected [224, 96]" in msg and "model.norm.weight: element type" in msg


def test_broken_files(tmp_path):
    folder = tiny.make_folder(tmp_path, tiny.TINY_A, 0)
    path = os.path.join(folder, "model.safetensors")
    data = open(path, "rb").read()
    open(path, "wb").write(data[: len(data) // 2])
    with pytest.raises(WeightError, match="truncated"):
        load_weights(folder, specs_of(tiny.TINY_A), torch.bfloat16, "cpu")
    open(path, "wb").write(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!")
    with pytest.raises(SafetensorsError, match="JSON"):
        ModelFiles(folder)
    os.remove(path)
    with pytest.raises(WeightError, match="no model.safetensors"):
        load_weights(folder, specs_of(tiny.TINY_A), torch.bfloat16, "cpu")


def test_counter_based_random_weights():
    """Element i of a tensor depends on (seed, name, i) alone: rows can be regenerated on their
    own, other tensors do not matter, and a scalar restatement of the formula gives the same bits."""
    from odin_infer_b200.parts.base import ParamSpec
    from odin_infer_b200.weights.random_init import host_tensor, random_tensor
    from tests.plain import random_weights_plain as R
    spec = ParamSpec("model.layers.3.mlp.up_proj.weight", (37, 24))
    full = random_tensor(spec, 5, torch.float32)
    assert torch.equal(host_tensor(spec.name, spec.shape, "matrix", 5, torch.float32, first_row=11, n_rows=9), full[11:20])
    bf = random_tensor(spec, 5, torch.bfloat16)
    assert torch.equal(bf, full.bfloat16())                      # the storage type is a rounding of the same values
    for i in (0, 1, 23, 24, 500, 37 * 24 - 1):
        v = R.element(5, spec.name, i, 0.0, 0.02)
        assert full.flatten()[i].item() == v and bf.flatten()[i].item() == R.to_bf16(v), i
    norm = random_tensor(ParamSpec("n.weight", (50,), init="norm"), 5, torch.float32)
    assert norm[7].item() == R.element(5, "n.weight", 7, 1.0, 0.1)
    assert not torch.equal(full, random_tensor(spec, 6, torch.float32))
    assert not torch.equal(full, random_tensor(ParamSpec("other", (37, 24)), 5, torch.float32))
    big = random_tensor(ParamSpec("big", (1 << 21,)), 1, torch.float32)          # across the host's chunks of 2^20
    assert abs(big.std().item() - 0.02) < 2e-4 and abs(big.mean().item()) < 1e-4 and big.abs().max().item() < 0.02 * 4.9
    assert big[(1 << 20) + 3].item() == R.element(1, "big", (1 << 20) + 3, 0.0, 0.02)

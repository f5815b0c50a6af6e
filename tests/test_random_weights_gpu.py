"""Random weights: the device's generator gives the host's bits, and an engine built from a seed
in memory computes what an engine loaded from the folder written with that seed computes."""
import pytest
import torch

from tests import tiny

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_device_generator_equals_host(dtype):
    from odin_infer_b200.parts.base import ParamSpec
    from odin_infer_b200.weights.random_init import host_tensor, random_tensor
    for name, shape, init in (("a.weight", (301, 72), "matrix"), ("n", (4099,), "norm"), ("big", (3, 1 << 20), "matrix")):
        dev = random_tensor(ParamSpec(name, shape, init=init), 9, dtype, device="cuda:0")
        assert dev.dtype == dtype and tuple(dev.shape) == shape
        assert torch.equal(dev.cpu(), host_tensor(name, shape, init, 9, dtype))
    # a few rows far into a tensor of the size of an 8B embedding table, without making the table on the host
    spec = ParamSpec("model.embed_tokens.weight", (151936, 4096))
    dev = random_tensor(spec, 5, dtype, device="cuda:0")
    for row in (0, 77777, 151935):
        assert torch.equal(dev[row:row + 2].cpu(), host_tensor(spec.name, spec.shape, "matrix", 5, dtype, first_row=row,
                                                               n_rows=min(2, 151936 - row)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_from_seed_equals_engine_from_written_folder(tmp_path, dtype):
    from odin_infer_b200 import Engine, Engine_Opts, StepEntry
    from odin_infer_b200.config import config_from_dict
    raw, seed = tiny.TINIES["E"]
    folder = tiny.make_folder(tmp_path, raw, seed)
    toks = tiny.random_tokens(90, raw["vocab_size"], 4)
    outs = []
    for make in (lambda o: Engine.load(folder, o), lambda o: Engine.random(config_from_dict(raw), seed, o)):
        e = make(Engine_Opts(max_ctx=128, max_batch=1, dtype=dtype, verbose=False))
        s = e.take_slot()
        outs.append(e.step([StepEntry(s, toks, list(range(len(toks))))]).cpu())
        e.destroy()
    assert torch.equal(outs[0], outs[1])

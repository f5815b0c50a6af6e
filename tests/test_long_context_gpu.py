"""Contexts of more than 8,192 tokens through the engine, against the plain implementation: a prompt
of 8,300 tokens in one step, its last tokens decoded one by one (decode attention with 16 key splits,
block tables of 130 pages, the largest context classes of the captured graphs), and a batch of
unequal lengths.  Random weights would hide a key that is lost among thousands: the per-head norms of
q and k are scaled up, so that each query's softmax rests on a handful of keys, most of them far away
(by a factor of 2 in 32-bit, where every lost key shows at 2e-5; by 1.5 in bfloat16, where the scores'
own rounding grows with their size; there the kernels' far-key tests plant the key that must be found)."""
import os

import numpy as np
import pytest
import torch

from tests import tiny, traces

pytestmark = pytest.mark.gpu

LONG = dict(architectures=["Qwen3ForCausalLM"], hidden_size=192, intermediate_size=320, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=1, head_dim=128, vocab_size=1000, rope_theta=1e6,
            rms_norm_eps=1e-6, tie_word_embeddings=True)
LENGTHS = {"r0": 8300, "r1": 4200, "r2": 700}
PEAK = {"float32": 2.0, "bfloat16": 1.5}   # factor on the weights of q_norm and k_norm: scores grow by its square


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def case(request, tmp_path_factory):
    from odin_infer_b200.weights import ModelFiles, write_safetensors
    from tests.plain import qwen3_plain
    dtype = request.param
    folder = tiny.make_folder(tmp_path_factory.mktemp("long_" + dtype), LONG, 31)
    files = ModelFiles(folder)
    tensors = {n: files.tensor(n).clone() for n in files.names()}
    for n in tensors:
        if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
            tensors[n] = (tensors[n].float() * PEAK[dtype]).to(tensors[n].dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], lambda n: tensors[n])
    reqs = {rid: tiny.random_tokens(n, LONG["vocab_size"], 900 + i) for i, (rid, n) in enumerate(LENGTHS.items())}
    wanted = {}
    for rid, toks in reqs.items():
        n = len(toks)
        rng = np.random.default_rng(n)
        fixed = {0, 63, 64, n // 2, n - 40, n - 33, n - 32, n - 31, n - 17, n - 2, n - 1, 8191, 8192, 8193, 4095, 4096}
        wanted[rid] = sorted({p for p in fixed if 0 <= p < n} | set(int(p) for p in rng.integers(0, n, 6)))
    cfg, w = qwen3_plain.read_model_folder(folder, torch.float64)
    refs = {rid: qwen3_plain.forward_whole(cfg, w, toks, positions=wanted[rid]).numpy() for rid, toks in reqs.items()}
    return folder, reqs, wanted, refs, dtype


def test_the_softmax_rests_on_few_far_keys(case):
    """The premise of this file, checked on the plain implementation's first layer: the largest
    attention weight of a late query is large, and the key it belongs to is far away."""
    from tests.plain import qwen3_plain as P
    folder, reqs, _, _, dtype = case
    cfg, w = P.read_model_folder(folder, torch.float64)
    toks = reqs["r0"]
    T, hd = len(toks), LONG["head_dim"]
    x = P.embedding(w["model.embed_tokens.weight"], toks)
    h = P.rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-6)
    cos, sin = P.rope_tables(T, hd, 1e6, torch.float64)
    q = P.rope(P.rmsnorm(P.linear(h, w["model.layers.0.self_attn.q_proj.weight"]).reshape(T, 4, hd),
                         w["model.layers.0.self_attn.q_norm.weight"], 1e-6), cos, sin)
    k = P.rope(P.rmsnorm(P.linear(h, w["model.layers.0.self_attn.k_proj.weight"]).reshape(T, 1, hd),
                         w["model.layers.0.self_attn.k_norm.weight"], 1e-6), cos, sin)
    late = torch.arange(T - 64, T)
    p = P.softmax_rows((q[late, 0] @ k[:, 0].t()) / hd ** 0.5 + torch.where(
        torch.arange(T)[None, :] <= late[:, None], 0.0, float("-inf")))
    top, where = p.max(dim=1)
    top5 = p.topk(5, dim=1).values.sum(1)
    assert top5.median() > (0.45 if dtype == "float32" else 0.1), "a handful of keys carry each query"
    assert ((late - where) > 1024).double().mean() > 0.5, "and most of them lie more than 1,024 tokens back"


def run(folder, dtype, recs, graphs=True, decodes=True):
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.engine.trace import replay
    n = traces.max_live_tokens(recs)
    e = Engine.load(folder, Engine_Opts(max_ctx=8320, max_tokens=n, dtype=dtype, verbose=False, cuda_graphs=graphs))
    try:
        got = traces.collect_places(recs, replay(e, recs))
        torch.cuda.synchronize()
        if dtype == "bfloat16":
            ops.gemm_tc_check()
            ops.attention_prefill_check()
            ops.attention_decode_check()
            if graphs and decodes:
                assert max(k[1] for k in e.graphs._graphs if k[0] != "prompt") >= 17, "the largest context classes ran"
        e.cache.check()
        return got
    finally:
        e.destroy()


def test_long_contexts_against_the_plain_implementation(case):
    folder, reqs, wanted, refs, dtype = case
    scheds = {"whole": traces.restrict(traces.whole(reqs), wanted),
              "last 40 one by one": traces.restrict(traces.tail_one_by_one(reqs, 40), wanted),
              "unequal batch": traces.restrict(traces.batches(reqs, 3, first_part=lambda n: n - 36), wanted)}
    if dtype == "bfloat16":
        scheds["unequal batch, no graphs"] = scheds["unequal batch"]
    for what, recs in scheds.items():
        got = run(folder, dtype, recs, graphs="no graphs" not in what, decodes=what != "whole")
        for rid, places in wanted.items():
            assert sorted(got[rid]) == places, (what, rid)
            for i, pos in enumerate(places):
                err = tiny.rel_err(got[rid][pos], refs[rid][i])
                assert err <= tiny.TOL[dtype], f"{what} {dtype}: request {rid} position {pos}: {err:.3e}"

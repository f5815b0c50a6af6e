"""Configurations drawn at random (fixed seeds) through the engine, against the plain implementation:
head sizes in steps of 16 up to 256 (most of them go to the kernels that take any size), up to 20
query heads on a kv head, widths and vocabularies that are no power of two and no multiple of 8."""
import numpy as np
import pytest

from tests import tiny, traces

pytestmark = pytest.mark.gpu


def draw(seed: int) -> dict:
    rng = np.random.default_rng(seed)
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256]))
    kv = int(rng.choice([1, 2, 3, 4]))
    g = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 16, 20]))
    if g * kv * hd > 4096:
        g = max(1, 4096 // (kv * hd))
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=int(rng.choice([40, 64, 72, 100, 128, 136, 200, 264, 520])),
                intermediate_size=int(rng.choice([56, 100, 128, 200, 264, 500, 1032])),
                num_hidden_layers=int(rng.integers(1, 4)), num_attention_heads=g * kv, num_key_value_heads=kv, head_dim=hd,
                vocab_size=int(rng.choice([97, 256, 301, 1000, 2051])), rope_theta=float(rng.choice([1e4, 5e5, 1e6])),
                rms_norm_eps=float(rng.choice([1e-6, 1e-5])), tie_word_embeddings=bool(rng.integers(0, 2)),
                max_position_embeddings=4096)


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106])
def test_a_configuration_drawn_at_random(seed, tmp_path):
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.engine.trace import replay
    raw = draw(seed)
    folder = tiny.make_folder(tmp_path, raw, seed)
    lens = np.random.default_rng(seed + 1).integers(1, 200, 4)
    reqs = {f"r{i}": tiny.random_tokens(int(n), raw["vocab_size"], 50 + i) for i, n in enumerate(lens)}
    refs = {rid: tiny.plain_logits(folder, toks) for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        for what, recs in (("whole", traces.whole(reqs)), ("last 32 one by one", traces.tail_one_by_one(reqs, 32)),
                           ("batches of 3", traces.batches(reqs, 3))):
            n = traces.max_live_tokens(recs)
            e = Engine.load(folder, Engine_Opts(max_ctx=n, max_tokens=n, dtype=dtype, verbose=False))
            try:
                got = traces.collect(recs, replay(e, recs))
                e.cache.check()
            finally:
                e.destroy()
            for rid in reqs:
                err = tiny.rel_err(got[rid], refs[rid])
                assert err <= tiny.TOL[dtype], f"{raw} {dtype} {what}: request {rid}: {err:.3e}"

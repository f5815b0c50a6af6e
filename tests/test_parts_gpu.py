"""Each part alone against the plain implementation's function for it, and a toy
architecture defined HERE (a mixer with state of its own, a feed-forward that routes each
token to one of its experts, a second position encoding that acts on the embedded tokens,
a layer that runs twice, a layer that reads another layer's cache, a windowed layer with
storage of its own), registered, built and stepped without touching the package's files."""
import dataclasses

import pytest
import torch

from tests import tiny, traces
from tests.plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, ref, rtol):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= rtol, f"relative error {err:.3e} > {rtol:.1e}"


def runtime(dtype):
    from odin_infer_b200.engine.runtime import Runtime
    return Runtime(DEV, dtype)


def make_step(mixers, entries_tokens, dtype, starts=None):
    """A cache and a StepBatch for the given mixers (one schedule entry each)."""
    from odin_infer_b200.cache import CacheManager
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    cache = CacheManager(64 * 16, 64 * 8)
    for m in mixers:
        cache.add_entry(m.cache_request(), m.state_bytes())
    cache.entry_writes = [True] * len(mixers)
    for g in cache.groups.values():
        g.attach_storage(torch.zeros(g.storage_shape(), dtype=dtype, device=DEV),
                         torch.zeros(g.storage_shape(), dtype=dtype, device=DEV))
    cache.state = torch.zeros(cache.max_slots, cache.state_bytes_per_slot, dtype=torch.uint8, device=DEV)
    entries, st = [], []
    for toks in entries_tokens:
        slot = cache.take_slot()
        st.append(cache.extend(slot, len(toks)))
        entries.append(StepEntry(slot, toks, list(range(len(toks)))))
    return cache, StepBatch(cache, entries, st, DEV)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 5e-3)])
def test_norm_part(dtype, tol):
    from odin_infer_b200.parts import PartSpec, build_part
    rt = runtime(dtype)
    norm = build_part("norm", PartSpec("rmsnorm", dict(width=72, eps=1e-5, weight="w")))
    assert [(p.name, p.shape, p.init) for p in norm.params()] == [("w", (72,), "norm")]
    w = (1 + 0.1 * torch.randn(72, device=DEV)).to(dtype)
    norm.bind({"w": w}, rt)
    x = torch.randn(5, 72, device=DEV)
    delta = torch.randn(5, 72, device=DEV)
    x0 = x.clone()
    h = norm.forward(rt, x, delta)
    assert h.dtype == dtype
    close(x, x0.double() + delta.double(), 1e-6)
    close(h, P.rmsnorm(x0.double().cpu() + delta.double().cpu(), w.double().cpu(), 1e-5), tol)


def test_rotary_part_tables():
    from odin_infer_b200.parts import PartSpec, build_part
    pe = build_part("position_encoding", PartSpec("rope", dict(rotary_dim=48, theta=5e5)))
    pe.prepare(runtime(torch.float32), 300)
    cos, sin, rot = pe.rotation()
    rc, rs = P.rope_tables(300, 48, 5e5, torch.float64)
    assert rot == 48 and cos.shape == (300, 24)
    close(cos, rc, 1e-6)
    close(sin.double().cpu() + 2, rs + 2, 1e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
def test_feed_forward_part(dtype, tol):
    from odin_infer_b200.parts import PartSpec, build_part
    rt = runtime(dtype)
    ffn = build_part("feed_forward", PartSpec("swiglu", dict(width=72, inner=200, names=dict(gate="g", up="u", down="d"))))
    assert sorted((p.name, p.shape) for p in ffn.params()) == [("d", (72, 200)), ("g", (200, 72)), ("u", (200, 72))]
    t = {"g": torch.randn(200, 72, device=DEV).to(dtype), "u": torch.randn(200, 72, device=DEV).to(dtype),
         "d": torch.randn(72, 200, device=DEV).to(dtype) * 0.1}
    ref_w = {k: v.double().cpu() for k, v in t.items()}
    ffn.bind(t, rt)
    h = torch.randn(9, 72, device=DEV).to(dtype)
    out = ffn.forward(rt, None, h)
    if out.dim() == 3:
        out = out.sum(0)
    close(out, P.swiglu_mlp(h.double().cpu(), ref_w["g"], ref_w["u"], ref_w["d"]), tol)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("geom", [(4, 2, 16), (4, 1, 64)])
def test_attention_part_prompt_then_single_tokens(dtype, tol, geom):
    from odin_infer_b200.engine.step import StepBatch, StepEntry
    from odin_infer_b200.parts import PartSpec, build_part
    n_q, n_kv, hd = geom
    width = 80
    rt = runtime(dtype)
    names = dict(q="q", k="k", v="v", o="o", q_norm="qn", k_norm="kn")
    att = build_part("mixer", PartSpec("gqa_attention", dict(width=width, n_q_heads=n_q, n_kv_heads=n_kv, head_dim=hd,
                                                             names=names, position_encoding="rope", eps=1e-6)))
    pe = build_part("position_encoding", PartSpec("rope", dict(rotary_dim=hd, theta=1e4)))
    pe.prepare(rt, 512)
    att.pe = pe
    torch.manual_seed(1)
    t = {"q": torch.randn(n_q * hd, width, device=DEV) * 0.2, "k": torch.randn(n_kv * hd, width, device=DEV) * 0.2,
         "v": torch.randn(n_kv * hd, width, device=DEV) * 0.2, "o": torch.randn(width, n_q * hd, device=DEV) * 0.2,
         "qn": 1 + 0.1 * torch.randn(hd, device=DEV), "kn": 1 + 0.1 * torch.randn(hd, device=DEV)}
    t = {k: v.to(dtype) for k, v in t.items()}
    ref_w = {("x." + {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "qn": "q_norm", "kn": "k_norm"}[k] + ".weight"):
             v.double().cpu() for k, v in t.items()}
    att.bind(dict(t), rt)
    n = 75
    h_all = torch.randn(n, width, device=DEV).to(dtype)
    cfg = dict(num_attention_heads=n_q, num_key_value_heads=n_kv, head_dim=hd, rms_norm_eps=1e-6)
    cos, sin = P.rope_tables(n, hd, 1e4, torch.float64)
    ref = P.attention_block(h_all.double().cpu(), ref_w, "x.", cfg, cos, sin)
    cache, step = make_step([att], [list(range(70))], dtype)
    out = att.forward(rt, step, h_all[:70], 0)
    out = out.sum(0) if out.dim() == 3 else out
    close(out, ref[:70], tol)
    slot = step.slots[0]
    for p in range(70, n):
        st = cache.extend(slot, 1)
        one = StepBatch(cache, [StepEntry(slot, [0], [0])], [st], DEV)
        o = att.forward(rt, one, h_all[p:p + 1], 0)
        o = o.sum(0) if o.dim() == 3 else o
        close(o[0], ref[p], tol)


def test_embedding_head_and_block_parts():
    from odin_infer_b200.parts import PartSpec, build_part
    rt = runtime(torch.float32)
    emb = build_part("embedding", PartSpec("token_table", dict(vocab_size=301, width=72, weight="e")))
    head = build_part("head", PartSpec("linear", dict(vocab_size=301, width=72, weight="lm", tied_to="e")))
    assert head.params()[0].alias_of == "e"
    table = torch.randn(301, 72, device=DEV)
    emb.bind({"e": table}, rt)
    head.bind({"lm": table}, rt)
    _, step = make_step([], [[5, 300, 0]], torch.float32)
    x = emb.forward(rt, step)
    assert torch.equal(x, table[[5, 300, 0]])
    close(head.forward(rt, step, x), x.double().cpu() @ table.double().cpu().t(), 2e-6)


# ------------------------------------------------------------------------------------
# A toy architecture, defined in this test only
# ------------------------------------------------------------------------------------
def register_toy():
    from odin_infer_b200.config import ModelConfig, register_architecture
    from odin_infer_b200.config.base import KeyReader
    from odin_infer_b200.parts import Mixer, ModelSpec, ParamSpec, PartSpec, ScheduleEntry, register_part
    from odin_infer_b200.parts.base import FeedForward, PositionEncoding

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(FeedForward):
        """Each token goes to the expert whose router logit is largest (32-bit logits, the first
        maximum wins) and gets that expert's SwiGLU."""

        def __init__(self, width: int, inner: int, experts: int, prefix: str):
            self.width, self.inner, self.experts, self.prefix = width, inner, experts, prefix
            self.router, self.w = None, []

        def params(self):
            out = [ParamSpec(f"{self.prefix}.router", (self.experts, self.width))]
            for e in range(self.experts):
                out += [ParamSpec(f"{self.prefix}.e{e}.{k}", shape) for k, shape in
                        (("gate", (self.inner, self.width)), ("up", (self.inner, self.width)), ("down", (self.width, self.inner)))]
            return out

        def bind(self, tensors, rt):
            self.router = tensors[f"{self.prefix}.router"]
            self.w = [tuple(tensors[f"{self.prefix}.e{e}.{k}"] for k in ("gate", "up", "down")) for e in range(self.experts)]

        def forward(self, rt, step, h):
            hf = h.float()
            choice = torch.argmax(hf @ self.router.float().t(), dim=1)
            out = torch.zeros(h.shape[0], self.width, dtype=torch.float32, device=h.device)
            for e, (g, u, d) in enumerate(self.w):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = hf[rows]
                    a = torch.nn.functional.silu(x @ g.float().t()) * (x @ u.float().t())
                    out[rows] = a.to(h.dtype).float() @ d.float().t()
            return out

    @register_part("position_encoding", "toy_learned")
    class LearnedPositions(PositionEncoding):
        """A table of one vector per position, added to the embedded tokens."""

        def __init__(self, width: int, max_positions: int, weight: str):
            self.width, self.max_positions, self.weight_name, self.table = width, max_positions, weight, None

        def params(self):
            return [ParamSpec(self.weight_name, (self.max_positions, self.width))]

        def bind(self, tensors, rt):
            self.table = tensors[self.weight_name]

        def on_embedding(self, rt, step, x):
            n = step.n_tokens
            x[:n] += self.table[step.tok_pos[:n].long()].float()

    @register_part("mixer", "toy_running_mean")
    class RunningMean(Mixer):
        """out_t = W mean(h_0 .. h_t): the state per sequence is the running sum and the count."""

        def __init__(self, width: int, weight: str):
            self.width, self.weight_name, self.w = width, weight, None

        def params(self):
            return [ParamSpec(self.weight_name, (self.width, self.width))]

        def bind(self, tensors, rt):
            self.w = tensors[self.weight_name]

        def state_bytes(self):
            return 4 * (self.width + 1)

        def forward(self, rt, step, h, entry):
            state = step.state(entry).view(torch.float32)      # [slots, width + 1]
            out = torch.zeros(h.shape[0], self.width, dtype=torch.float32, device=h.device)
            starts = step.seq_start_host          # first token row of each sequence, and the end
            for b in range(step.n_seqs):
                a, e = starts[b], starts[b + 1]
                slot = step.slots[b]
                sums = state[slot, :self.width] + torch.cumsum(h[a:e].float(), 0)
                cnt = state[slot, self.width] + torch.arange(1, e - a + 1, device=h.device, dtype=torch.float32)
                out[a:e] = (sums / cnt[:, None]) @ self.w.float().t()
                state[slot, :self.width] = sums[-1]
                state[slot, self.width] = cnt[-1]
            return out

    # ---- the same three parts written to the contract of `graph_safe`: indices from the step's
    # device tensors only, launches sized by the padded row count, rows of sequence -1 skipped
    @register_part("feed_forward", "toy_top1_experts_dense")
    class Top1ExpertsDense(Top1Experts):
        """Every expert runs on every row and the chosen one's result is kept: no shape depends on the data."""
        graph_safe = True

        def forward(self, rt, step, h):
            hf = h.float()
            choice = torch.argmax(hf @ self.router.float().t(), dim=1)
            out = torch.zeros(h.shape[0], self.width, dtype=torch.float32, device=h.device)
            for e, (g, u, d) in enumerate(self.w):
                a = torch.nn.functional.silu(hf @ g.float().t()) * (hf @ u.float().t())
                out = torch.where((choice == e)[:, None], a.to(h.dtype).float() @ d.float().t(), out)
            return out

    @register_part("position_encoding", "toy_learned_by_rows")
    class LearnedPositionsByRows(LearnedPositions):
        graph_safe = True

        def on_embedding(self, rt, step, x):
            n = x.shape[0]
            real = (step.tok_seq[:n] >= 0)[:, None]
            x += torch.where(real, self.table[step.tok_pos[:n].long()].float(), torch.zeros((), device=x.device))

    @register_part("mixer", "toy_running_mean_by_rows")
    class RunningMeanByRows(RunningMean):
        """The same running mean with every index taken from the device: a segmented cumulative sum
        over the rows (sum up to a row minus the sum before its sequence's first row), the state
        gathered by `seq_slots`, and written back by the last row of each sequence as an increment
        (rows that are not the last, and padding rows, add zero)."""
        graph_safe = True

        def forward(self, rt, step, h, entry):
            state = step.state(entry).view(torch.float32)      # [slots, width + 1]
            n, w = h.shape[0], self.width
            seq = step.tok_seq[:n].long()
            real = seq >= 0
            seq0 = seq.clamp(min=0)
            hf = torch.where(real[:, None], h.float(), torch.zeros((), device=h.device))
            cs = torch.cumsum(hf, 0)
            first = step.seq_start.long()[seq0]                 # first row of the row's sequence
            before = torch.where((first > 0)[:, None], cs[(first - 1).clamp(min=0)], torch.zeros((), device=h.device))
            old = state[step.seq_slots.long()[seq0]]            # [n, width + 1]
            sums = old[:, :w] + (cs - before)
            cnt = old[:, w] + (torch.arange(n, device=h.device) - first + 1).float()
            out = torch.where(real[:, None], (sums / cnt[:, None]) @ self.w.float().t(), torch.zeros((), device=h.device))
            last = real & (torch.arange(1, n + 1, device=h.device) == step.seq_start.long()[seq0 + 1])
            inc = torch.cat([sums, cnt[:, None]], 1) - old
            state.index_add_(0, step.seq_slots.long()[seq0], torch.where(last[:, None], inc, torch.zeros((), device=h.device)))
            return out

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 0
        vocab: int = 0
        heads: int = 0
        kv_heads: int = 0
        head_dim: int = 0
        inner: int = 0
        window: int = 0
        experts: int = 0
        max_positions: int = 0
        by_rows: int = 0     # 1: the parts written for CUDA graphs
        eps: float = 1e-6
        theta: float = 1e4

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            r = KeyReader(raw, where)
            vals = {k: r.get(k, int) for k in ("width", "vocab", "heads", "kv_heads", "head_dim", "inner", "window",
                                               "experts", "max_positions")}
            vals["by_rows"] = r.get("by_rows", int, 0)
            r.finish()
            return cls(architecture=raw["architectures"][0], **vals)

        def to_dict(self):
            d = dataclasses.asdict(self)
            d["architectures"] = [d.pop("architecture")]
            return d

    def build(cfg):
        def attn(prefix, window=0, shared=False):
            names = {k: f"{prefix}.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")}
            return PartSpec("gqa_attention", dict(width=cfg.width, n_q_heads=cfg.heads, n_kv_heads=cfg.kv_heads,
                                                  head_dim=cfg.head_dim, names=names, position_encoding="rope",
                                                  eps=cfg.eps, window=window, kv_shared=shared))

        def block(l, mixer, routed=False):
            ffn = PartSpec("swiglu", dict(width=cfg.width, inner=cfg.inner,
                                          names={k: f"l{l}.ffn.{k}" for k in ("gate", "up", "down")}))
            if routed:
                ffn = PartSpec("toy_top1_experts_dense" if cfg.by_rows else "toy_top1_experts", dict(width=cfg.width, inner=cfg.inner, experts=cfg.experts, prefix=f"l{l}.moe"))
            n1 = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight=f"l{l}.n1"))
            n2 = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight=f"l{l}.n2"))
            return PartSpec("prenorm", dict(mixer=mixer, feed_forward=ffn, norm_mixer=n1, norm_feed_forward=n2))
        layers = (block(0, attn("l0.att")), block(1, attn("l1.att", window=cfg.window)),
                  block(2, attn("l2.att", shared=True)),
                  block(3, PartSpec("toy_running_mean_by_rows" if cfg.by_rows else "toy_running_mean",
                                    dict(width=cfg.width, weight="l3.mix")), routed=True))
        return ModelSpec(
            width=cfg.width, vocab_size=cfg.vocab,
            embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, width=cfg.width, weight="emb")),
            position_encodings={"rope": PartSpec("rope", dict(rotary_dim=cfg.head_dim, theta=cfg.theta)),
                                "learned": PartSpec("toy_learned_by_rows" if cfg.by_rows else "toy_learned", dict(width=cfg.width, max_positions=cfg.max_positions,
                                                                        weight="pos"))},
            layers=layers,
            # layer 0 runs twice (each run keeps its own cache); layer 2 reads the cache of the first run
            schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, reads_cache_of=0), ScheduleEntry(3)),
            final_norm=PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight="final")),
            head=PartSpec("linear", dict(vocab_size=cfg.vocab, width=cfg.width, weight="head", tied_to="emb")))

    register_architecture("ToyForCausalLM", ToyConfig, build)
    return ToyConfig


TOY = dict(architectures=["ToyForCausalLM"], width=64, vocab=200, heads=4, kv_heads=2, head_dim=16, inner=96, window=40,
           experts=3, max_positions=256)


def toy_plain(w, cfg, tokens):
    """The toy model, whole sequence, with the plain implementation's functions.  Returns the logits and,
    per position, by how much the chosen expert's router logit leads (a small lead may go the other
    way under rounding)."""
    T = len(tokens)
    hq, hkv, hd, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], 1e-6
    cos, sin = P.rope_tables(T, hd, 1e4, torch.float64)

    def qkv(p, x, need_kv=True):
        q = P.rope(P.rmsnorm(P.linear(x, w[p + ".q"]).reshape(T, hq, hd), w[p + ".q_norm"], eps), cos, sin)
        if not need_kv:
            return q, None, None
        k = P.rope(P.rmsnorm(P.linear(x, w[p + ".k"]).reshape(T, hkv, hd), w[p + ".k_norm"], eps), cos, sin)
        return q, k, P.linear(x, w[p + ".v"]).reshape(T, hkv, hd)

    def ffn(l, x):
        return P.swiglu_mlp(P.rmsnorm(x, w[f"l{l}.n2"], eps), w[f"l{l}.ffn.gate"], w[f"l{l}.ffn.up"], w[f"l{l}.ffn.down"])
    x = P.embedding(w["emb"], tokens) + w["pos"][:T]
    # entry 0: layer 0
    q, k0, v0 = qkv("l0.att", P.rmsnorm(x, w["l0.n1"], eps))
    x = x + P.linear(P.causal_attention(q, k0, v0), w["l0.att.o"])
    x = x + ffn(0, x)
    # entry 1: layer 1, windowed
    q, k, v = qkv("l1.att", P.rmsnorm(x, w["l1.n1"], eps))
    x = x + P.linear(P.causal_attention(q, k, v, window=cfg["window"]), w["l1.att.o"])
    x = x + ffn(1, x)
    # entry 2: layer 0 again, on new activations
    q, k, v = qkv("l0.att", P.rmsnorm(x, w["l0.n1"], eps))
    x = x + P.linear(P.causal_attention(q, k, v), w["l0.att.o"])
    x = x + ffn(0, x)
    # entry 3: layer 2 reads the keys and values of entry 0
    q, _, _ = qkv("l2.att", P.rmsnorm(x, w["l2.n1"], eps), need_kv=False)
    x = x + P.linear(P.causal_attention(q, k0, v0), w["l2.att.o"])
    x = x + ffn(2, x)
    # entry 4: running mean mixer
    h = P.rmsnorm(x, w["l3.n1"], eps)
    mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=h.dtype)[:, None]
    x = x + P.linear(mean, w["l3.mix"])
    h = P.rmsnorm(x, w["l3.n2"], eps)
    router = P.linear(h, w["l3.moe.router"])
    top2 = torch.topk(router, 2, dim=1).values
    choice = torch.argmax(router, dim=1)
    routed = torch.zeros_like(x)
    for t in range(T):
        e = int(choice[t])
        routed[t] = P.swiglu_mlp(h[t:t + 1], w[f"l3.moe.e{e}.gate"], w[f"l3.moe.e{e}.up"], w[f"l3.moe.e{e}.down"])[0]
    x = x + routed
    return P.linear(P.rmsnorm(x, w["final"], eps), w["emb"]), (top2[:, 0] - top2[:, 1]) / router.abs().max()


@pytest.mark.parametrize("by_rows", [0, 1])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registers_builds_and_steps(tmp_path, dtype, by_rows):
    """With the engine's default options.  by_rows = 0: the parts written the natural way (host
    copies of slots and row ranges, shapes that follow the data): the engine runs such a model
    eagerly.  by_rows = 1: the same parts written to the contract of `graph_safe`: the bfloat16
    steps are captured and replayed, also across a page border and a border of context classes."""
    register_toy()
    from odin_infer_b200 import Engine, Engine_Opts
    from odin_infer_b200.config import config_from_dict
    from odin_infer_b200.engine.trace import replay
    from odin_infer_b200.weights import write_random_model
    raw = dict(TOY, by_rows=by_rows, max_positions=640 if by_rows else 256)
    folder = write_random_model(str(tmp_path / "toy"), config_from_dict(raw), seed=21)
    _, w = P.read_model_folder(folder, torch.float64)
    assert "l2.att.k" not in w and "head" not in w and "l3.mix" in w      # shared kv: no k/v; tied head
    assert "l3.moe.e2.down" in w and "l3.ffn.gate" not in w and tuple(w["pos"].shape) == (raw["max_positions"], 64)
    lengths = [3, 70, 150, 41] + ([530] if by_rows else [])              # 530: from context class 1 into class 2
    reqs = {f"r{i}": tiny.random_tokens(n, TOY["vocab"], 50 + i) for i, n in enumerate(lengths)}
    refs, leads = {}, {}
    for rid, toks in reqs.items():
        logits, lead = toy_plain(w, TOY, toks)
        refs[rid], leads[rid] = logits.numpy(), lead.numpy()
    assert sum(int((l > 0.05).sum()) for l in leads.values()) > 150, "most positions have a clear choice of expert"
    tol = tiny.TOL[dtype]
    for what, recs in (("whole", traces.whole(reqs)), ("tail", traces.tail_one_by_one(reqs, 32)),
                       ("batches", traces.batches(reqs, 2)), ("joining", traces.joining(reqs, 3))):
        n = traces.max_live_tokens(recs)
        e = Engine.load(folder, Engine_Opts(max_ctx=n, max_tokens=n, dtype=dtype, verbose=False))
        assert len(e.cache.groups) == 2                     # all keys / a window of them: storage of their own
        assert e.cache.line_of[3] == e.cache.line_of[0]     # the reading entry has no line of its own
        assert e.cache.line_of[2] != e.cache.line_of[0]     # the second run of layer 0 has
        assert e.cache.state_bytes_per_slot >= 4 * 65
        assert (e.graphs is not None) == (bool(by_rows) and dtype == "bfloat16")
        got = traces.collect(recs, replay(e, recs))
        e.cache.check()
        if e.graphs is not None:
            assert len(e.graphs._graphs) >= (1 if what == "whole" else 2), "steps were captured and replayed"
        for rid, ref in refs.items():
            for pos in range(ref.shape[0]):
                if leads[rid][pos] <= 0.05:  # a near tie between experts: rounding may decide it the other way
                    continue
                err = tiny.rel_err(got[rid][pos], ref[pos])
                assert err <= tol, f"toy {what} {dtype} by_rows={by_rows}: request {rid} first differs at position {pos}: {err:.3e}"
        e.destroy()

"""Each kernel alone against a plain float32/float64 torch reference of the same
operation, at sizes other than the engine's (odd widths, head sizes 16..160, groups
1..5, vocabularies that are no power of two)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, k=1):
    return (2e-6 if dtype == torch.float32 else 1e-2) * max(1.0, math.sqrt(k) / 8)


def close(got, ref, rtol):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err <= rtol, f"relative error {err:.3e} > {rtol:.1e}"


@pytest.mark.parametrize("table_dtype", DTYPES)
def test_embed(table_dtype):
    from odin_infer_b200.csrc import ops
    V, d = 301, 72
    table = torch.randn(V, d, device=DEV).to(table_dtype)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, d, device=DEV)
    ops.embed(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("w_dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 1000, 4096])
def test_add_rmsnorm(d, w_dtype, out_dtype):
    from odin_infer_b200.csrc import ops
    n, eps = 7, 1e-5
    x = torch.randn(n, d, device=DEV)
    delta = torch.randn(3, n, d, device=DEV)
    w = (1 + 0.1 * torch.randn(d, device=DEV)).to(w_dtype)
    x0 = x.clone()
    out = torch.empty(n, d, device=DEV, dtype=out_dtype)
    ops.add_rmsnorm(x, delta, w, eps, out)
    xr = x0.double() + delta.double().sum(0)
    ref = w.double() * (xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + eps))
    close(x, xr, 1e-6)
    close(out, ref, 2e-6 if out_dtype == torch.float32 else 5e-3)
    # gather of rows, no write-back, bf16 delta
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    d2 = torch.randn(n, d, device=DEV).bfloat16()
    x1 = x.clone()
    out2 = torch.empty(3, d, device=DEV, dtype=out_dtype)
    ops.add_rmsnorm(x, d2, w, eps, out2, rows)
    assert torch.equal(x, x1)
    xr2 = (x1.double() + d2.double())[rows.long()]
    ref2 = w.double() * (xr2 / torch.sqrt((xr2 * xr2).mean(-1, keepdim=True) + eps))
    close(out2, ref2, 2e-6 if out_dtype == torch.float32 else 5e-3)
    # no delta at all
    out3 = torch.empty(n, d, device=DEV, dtype=out_dtype)
    ops.add_rmsnorm(x, None, w, eps, out3)
    ref3 = w.double() * (x1.double() / torch.sqrt((x1.double() ** 2).mean(-1, keepdim=True) + eps))
    close(out3, ref3, 2e-6 if out_dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("case", [(1, 4096, 4), (8, 4096, 4), (128, 4096, 3), (129, 4096, 3), (200, 4096, 5), (8, 5120, 4),
                                  (64, 8192, 2), (8, 8200, 2), (16, 4100, 9)])
def test_add_rmsnorm_wide_rows(case):
    """Few wide rows, bfloat16 out, as in a decode step: the kernel of 1,024 threads with the row in registers
    (one or two groups of four a thread, up to 128 rows and a width of 8192) and the kernel of 512 threads on either
    side of it; every row with a scale of its own, one to nine parts to add; and the same bits as the 32-bit-out
    kernel's x, whose sum runs in the same order."""
    from odin_infer_b200.csrc import ops
    n, d, parts = case
    eps = 1e-6
    torch.manual_seed(n + d)
    x = torch.randn(n, d, device=DEV) * torch.linspace(0.1, 30.0, n, device=DEV)[:, None]
    x0 = x.clone()
    w = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    delta = torch.randn(parts, n, d, device=DEV) * 3
    out = torch.full((n, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(x, delta, w, eps, out)
    xr = x0.double() + delta.double().sum(0)
    ref = w.double() * (xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + eps))
    close(x, xr, 1e-6)
    assert (out.double() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    x32 = x0.clone()
    ops.add_rmsnorm(x32, delta, w, eps, torch.empty(n, d, device=DEV))
    assert torch.equal(x32, x), "the parts are added in another order than in the 32-bit kernel"
    # gather of rows (the final norm of a decode step): x untouched, padding rows give zeros
    rows = torch.tensor([n - 1, -1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.full((3, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    x1 = x.clone()
    ops.add_rmsnorm(x, None, w, eps, out2, rows)
    assert torch.equal(x, x1)
    ref2 = w.double() * (x1.double() / torch.sqrt((x1.double() ** 2).mean(-1, keepdim=True) + eps))
    assert (out2[0].double() - ref2[n - 1]).abs().max().item() <= 2 ** -7 * ref2[n - 1].abs().max().item()
    assert (out2[2].double() - ref2[0]).abs().max().item() <= 2 ** -7 * ref2[0].abs().max().item()
    assert torch.equal(out2[1], torch.zeros_like(out2[1]))


@pytest.mark.parametrize("delta_dtype", [None, torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [72, 1000, 2048, 4096, 5120, 8200])
def test_add_rmsnorm_many_rows(d, delta_dtype):
    """More than 256 rows, bfloat16 out: the prompt's variant (the row in registers; widths up to 8192,
    beyond that the kernel of few rows), each row with a scale of its own so that a row read from the
    wrong place shows."""
    from odin_infer_b200.csrc import ops
    n, eps = 301, 1e-6
    torch.manual_seed(d)
    x = torch.randn(n, d, device=DEV) * torch.linspace(0.1, 30.0, n, device=DEV)[:, None]
    x0 = x.clone()
    w = (1 + 0.1 * torch.randn(d, device=DEV)).bfloat16()
    delta = None if delta_dtype is None else (torch.randn(2, n, d, device=DEV) * 3).to(delta_dtype)
    out = torch.full((n, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(x, delta, w, eps, out)
    xr = x0.double() if delta is None else x0.double() + delta.double().sum(0)
    ref = w.double() * (xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + eps))
    close(x, xr, 1e-6)
    assert (out.double() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from odin_infer_b200.csrc import ops
    T, I = 5, 203
    gu = (3 * torch.randn(T, 2 * I, device=DEV)).to(dtype)
    out = torch.empty(T, I, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, :I].double(), gu[:, I:].double()
    close(out, g * torch.sigmoid(g) * u, 2e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("case", [(8, 12288, 3), (64, 1000, 2), (3, 204, 7), (5, 203, 2), (1, 64, 1)])
def test_swiglu_of_partial_sums(case):
    """The 32-bit partial sums of a split product in, bfloat16 out (the decode step's use): the vector
    kernel where the width allows it, the scalar one else, both against the formula in float64."""
    from odin_infer_b200.csrc import ops
    T, I, parts = case
    torch.manual_seed(I)
    gu = torch.randn(parts, T, 2 * I, device=DEV) * (2.0 / math.sqrt(parts))
    out = torch.full((T, I), float("nan"), device=DEV, dtype=torch.bfloat16)
    ops.swiglu(gu, out)
    sums = gu.double().sum(0)
    g, u = sums[:, :I], sums[:, I:]
    close(out, g * torch.sigmoid(g) * u, 5e-3)


@pytest.mark.parametrize("shape", [(1, 5, 3), (7, 130, 72), (65, 64, 16), (130, 301, 200), (3, 1000, 1032)])
@pytest.mark.parametrize("combo", [(torch.float32,) * 3, (torch.bfloat16,) * 3,
                                   (torch.bfloat16, torch.bfloat16, torch.float32),
                                   (torch.bfloat16, torch.float32, torch.bfloat16)])
def test_gemm_plain_ladder(shape, combo):
    """Structured inputs first (all ones gives K; an identity copies; rows and columns
    that differ), then random ones, as the reference's matrix-product harness does
    (gemm_harness/gemm_test.odin:1063-1072)."""
    from odin_infer_b200.csrc import ops
    M, N, K = shape
    ta, tw, tc = combo

    def run(a, w):
        out = torch.empty(M, N, device=DEV, dtype=tc)
        ops.gemm_plain(a.to(ta), w.to(tw), out)
        return out
    exact = 1e-7 if tc == torch.float32 else 4e-3
    close(run(torch.ones(M, K, device=DEV), torch.ones(N, K, device=DEV)), torch.full((M, N), float(K)), exact)
    eye = torch.eye(N, K, device=DEV)
    a = torch.randn(M, K, device=DEV).to(ta).float()
    close(run(a, eye), (a.double() @ eye.double().t()), exact)
    rows = torch.arange(M, device=DEV, dtype=torch.float32)[:, None].expand(M, K) % 7
    cols = (torch.arange(N, device=DEV, dtype=torch.float32)[:, None].expand(N, K) % 5) * 0.25
    close(run(rows, cols), rows.double() @ cols.double().t(), exact)
    a = torch.randn(M, K, device=DEV).to(ta)
    w = torch.randn(N, K, device=DEV).to(tw)
    # 32-bit: rounding of a K-term sum grows like sqrt(K) * 2^-24
    close(run(a, w), a.double() @ w.double().t(), (1e-7 * math.sqrt(K) if tc == torch.float32 else 5e-3))


def paged_cache(n_seqs, lengths, n_kv, hd, dtype, shuffle=True):
    """A cache whose pages are handed out in a scrambled order."""
    PAGE = 64
    pages_per = [(n + PAGE - 1) // PAGE for n in lengths]
    total = sum(pages_per) + 3
    order = torch.randperm(total).tolist() if shuffle else list(range(total))
    bt = torch.full((n_seqs, max(pages_per)), -1, dtype=torch.int32)
    it = iter(order)
    for s, n in enumerate(pages_per):
        for p in range(n):
            bt[s, p] = next(it)
    k = torch.full((total, n_kv, PAGE, hd), float("nan"), device=DEV, dtype=dtype)
    v = torch.full((total, n_kv, PAGE, hd), float("nan"), device=DEV, dtype=dtype)
    return k, v, bt.to(DEV)


def rope_ref(v, pos, rot, theta):
    half = rot // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1) / np.power(np.float32(theta), i / np.float32(half))).astype(np.float32)
    ang = torch.from_numpy((np.asarray(pos, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32).astype(np.float64))
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x, y = v[..., :half], v[..., half:rot]
    return torch.cat([x * c - y * s, x * s + y * c, v[..., rot:]], dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("geom", [(4, 2, 16, 16), (6, 2, 32, 32), (5, 1, 48, 48), (8, 8, 128, 128), (3, 3, 160, 64),
                                  (2, 1, 64, 0)])
def test_head_prep_and_attention_plain(geom, dtype):
    """q/k norm + rotation + cache write, then attention over the scrambled pages, for
    sequences that continue from a non-zero position, against a direct computation."""
    from odin_infer_b200.csrc import ops
    from odin_infer_b200.parts.position import RotaryEncoding
    from odin_infer_b200.engine.runtime import Runtime
    n_q, n_kv, hd, rot = geom
    theta, eps = 1e4, 1e-5
    lengths = [70, 1, 130]
    torch.manual_seed(n_q * 100 + hd)
    k_cache, v_cache, bt = paged_cache(3, lengths, n_kv, hd, dtype)
    rt = Runtime(DEV, dtype)
    pe = RotaryEncoding(max(rot, 2), theta)
    pe.prepare(rt, 256)
    qn = (1 + 0.1 * torch.randn(hd, device=DEV))
    kn = (1 + 0.1 * torch.randn(hd, device=DEV))
    width = (n_q + 2 * n_kv) * hd
    all_q, all_k, all_v = {}, {}, {}
    # two steps: first all but the last 3 tokens of each sequence (at least 1), then the rest
    cuts = [max(1, n - 3) for n in lengths]
    full = [torch.randn(n, width, device=DEV).to(dtype) for n in lengths]
    outs = [[] for _ in lengths]
    for part in range(2):
        seqs = [(s, (0, cuts[s]) if part == 0 else (cuts[s], lengths[s])) for s in range(3)]
        seqs = [(s, r) for s, r in seqs if r[1] > r[0]]
        qkv = torch.cat([full[s][a:b] for s, (a, b) in seqs]).clone()
        tok_pos = torch.tensor([p for s, (a, b) in seqs for p in range(a, b)], dtype=torch.int32, device=DEV)
        tok_seq = torch.tensor([s for s, (a, b) in seqs for _ in range(a, b)], dtype=torch.int32, device=DEV)
        ops.head_prep(qkv, n_q, n_kv, hd, qn, kn, eps, pe.cos, pe.sin, rot, tok_pos, tok_seq, bt, k_cache, v_cache)
        q = qkv[:, :n_q * hd]
        out = torch.empty(qkv.shape[0], n_q * hd, device=DEV, dtype=dtype)
        ops.attention_plain(q, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0)
        r = 0
        for s, (a, b) in seqs:
            outs[s].append(out[r:r + b - a])
            r += b - a
    for s, n in enumerate(lengths):
        x = full[s].double().cpu().view(n, n_q + 2 * n_kv, hd)
        def norm(v, w):
            return w.double().cpu() * (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps))
        pos = list(range(n))
        qr = rope_ref(norm(x[:, :n_q], qn), pos, rot, theta) if rot else norm(x[:, :n_q], qn)
        kr = rope_ref(norm(x[:, n_q:n_q + n_kv], kn), pos, rot, theta) if rot else norm(x[:, n_q:n_q + n_kv], kn)
        if dtype == torch.bfloat16:  # what the kernel stores
            qr, kr = qr.bfloat16().double(), kr.bfloat16().double()
        vr = x[:, n_q + n_kv:]
        ref = torch.zeros(n, n_q, hd, dtype=torch.float64)
        mask = torch.tril(torch.ones(n, n, dtype=torch.bool))
        for h in range(n_q):
            kh = h // (n_q // n_kv)
            sc = (qr[:, h] @ kr[:, kh].t()) / math.sqrt(hd)
            sc = sc.masked_fill(~mask, float("-inf"))
            ref[:, h] = torch.softmax(sc, -1) @ vr[:, kh]
        got = torch.cat(outs[s]).double().cpu().view(n, n_q, hd)
        close(got, ref, 3e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("geom", [(8, 2, 128), (6, 3, 64)])
@pytest.mark.parametrize("parts", [0, 2])
def test_head_prep_many_tokens_equals_few_at_a_time(geom, parts):
    """Prompts take a variant of the kernel that handles four tokens per warp: the same bits as the
    one-token variant run on pieces of the rows; a row count that is no multiple of four, a
    padding row, positions that differ per row."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    T, width = 517, (n_q + 2 * n_kv) * hd
    torch.manual_seed(hd + parts)
    lengths = [300, 217]
    k_cache, v_cache, bt = paged_cache(2, lengths, n_kv, hd, torch.bfloat16)
    tok_seq = torch.tensor([0] * 300 + [1] * 217, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(list(range(300)) + list(range(217)), dtype=torch.int32, device=DEV)
    tok_seq[77] = -1  # a padding row
    qkv = torch.randn(T, width, device=DEV).bfloat16() if parts == 0 else torch.randn(parts, T, width, device=DEV)
    qn = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    kn = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    ang = torch.arange(320, device=DEV, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV) / (hd // 2)))[None, :]
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    ka, va, kb, vb = k_cache.clone(), v_cache.clone(), k_cache.clone(), v_cache.clone()
    q_all = torch.full((T, n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.head_prep(qkv, n_q, n_kv, hd, qn, kn, 1e-6, cos, sin, hd, tok_pos, tok_seq, bt, ka, va, q_out=q_all)
    q_pieces = torch.full_like(q_all, 7.0)
    for a in range(0, T, 100):
        b = min(T, a + 100)
        piece = qkv[a:b].contiguous() if parts == 0 else qkv[:, a:b].contiguous()
        ops.head_prep(piece, n_q, n_kv, hd, qn, kn, 1e-6, cos, sin, hd, tok_pos[a:b].contiguous(),
                      tok_seq[a:b].contiguous(), bt, kb, vb, q_out=q_pieces[a:b])
    assert torch.equal(q_all, q_pieces)
    assert torch.equal(q_all[77], torch.full_like(q_all[77], 7.0)), "a padding row must not be written"
    # NaN marks the places that nobody wrote: they must agree too
    assert torch.equal(torch.nan_to_num(ka.float(), nan=-1.0), torch.nan_to_num(kb.float(), nan=-1.0))
    assert torch.equal(torch.nan_to_num(va.float(), nan=-1.0), torch.nan_to_num(vb.float(), nan=-1.0))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_respects_window(dtype):
    """One key far back among hundreds is made to stand out (its score dominates), so a
    kernel that skips or misplaces a page, or reads beyond the window, shows."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd, n = 4, 2, 32, 300
    torch.manual_seed(3)
    k_cache, v_cache, bt = paged_cache(1, [n], n_kv, hd, dtype)
    keys = 0.1 * torch.randn(n, n_kv, hd, device=DEV)
    vals = torch.randn(n, n_kv, hd, device=DEV)
    far = 67  # second page
    q = 0.1 * torch.randn(1, n_q, hd, device=DEV)
    keys[far] = 0.0
    keys[far, :, 0] = 40.0
    q[0, :, 0] = 40.0 / math.sqrt(hd) * 2
    for p in range(n):
        page = int(bt[0, p // 64])
        k_cache[page, :, p % 64] = keys[p].to(dtype)
        v_cache[page, :, p % 64] = vals[p].to(dtype)
    tok_pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    tok_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    qf = q.reshape(1, n_q * hd).to(dtype)
    out = torch.empty(1, n_q * hd, device=DEV, dtype=dtype)
    ops.attention_plain(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0)
    got = out.float().view(n_q, hd)
    for h in range(n_q):
        close(got[h], vals[far, h // 2].to(dtype).float(), 2e-2)
    # with a window that ends after the far key, it must not be seen
    ops.attention_plain(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, n - 1 - far)
    got_w = out.float().view(n_q, hd)
    assert (got_w - vals[far, 0].to(dtype).float()).abs().max() > 0.1
    # and with a window that just includes it, it is seen again
    ops.attention_plain(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, n - far)
    close(out.float().view(n_q, hd)[0], vals[far, 0].to(dtype).float(), 2e-2)


def test_argmax_and_sampling():
    from odin_infer_b200.csrc import ops
    from tests.plain import qwen3_plain as P
    B, V = 5, 1003
    torch.manual_seed(0)
    logits = torch.randn(B, V, device=DEV) * 3
    logits[1, 17] = logits[1, 900] = 50.0  # a tie: the first wins
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert out.tolist() == [P.argmax_first(logits[b].tolist()) for b in range(B)]
    assert out[1].item() == 17
    keep = logits.clone()
    # temperature draw: the token must be the one the plain CDF walk finds (or its neighbour
    # when the coin falls within rounding of a boundary)
    coins = torch.tensor([0.0, 0.25, 0.5, 0.75, 0.999], device=DEV)
    ops.sample(logits, 0.8, 1.0, coins, out)
    assert torch.equal(logits, keep), "sampling must leave the logits as they are"
    for b in range(B):
        p = P.temperature_probs(logits[b].double().cpu(), 0.8)
        cdf = torch.cumsum(p, 0)
        i = out[b].item()
        lo = cdf[i - 1].item() if i > 0 else 0.0
        assert lo - 1e-5 <= coins[b].item() < cdf[i].item() + 1e-5, (b, i)
    # top-p: the drawn token is always in the kept set; with a tiny top_p it is the argmax
    # (no tied logits here: which of two equal tokens a sort keeps is not defined)
    logits[1, 900] = 49.0
    for tp in (0.3, 0.9):
        for c in (0.0, 0.37, 0.99):
            ops.sample(logits, 1.0, tp, torch.full((B,), c, device=DEV), out)
            for b in range(B):
                p = P.temperature_probs(logits[b].double().cpu(), 1.0)
                assert out[b].item() in P.top_p_keep(p, tp)
    ops.sample(logits, 1.0, 1e-4, torch.full((B,), 0.9, device=DEV), out)
    assert out.tolist() == logits.argmax(-1).tolist()
    # the draws follow the distribution
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device=DEV).repeat(4000, 1)
    cs = torch.rand(4000, device=DEV)
    o = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(small, 1.0, 1.0, cs, o)
    freq = torch.bincount(o.long(), minlength=4).double() / 4000
    assert (freq.cpu() - torch.softmax(small[0].double().cpu(), 0)).abs().max() < 0.03


@pytest.mark.parametrize("V", [1003, 151936])
def test_top_p_draws_the_references_token(V):
    """With top-p the reference walks the kept tokens in order of falling probability with the coin
    scaled by their sum: for the same coin the kernel gives that very token (a coin within rounding
    of a boundary may give the neighbour in that order), also with exact ties inside the kept set and
    at the cut, where index order decides."""
    from odin_infer_b200.csrc import ops
    from tests.plain import qwen3_plain as P
    torch.manual_seed(V)
    rows = [torch.randn(V) * 4, torch.randn(V) * 1.5, torch.randn(V) * 0.3, torch.zeros(V)]
    rows[3][:8] = torch.tensor([5.0, 5.0, 4.0, 5.0, 4.0, 3.0, 3.0, 3.0])      # ties of three, two, three
    rows.append(torch.cat([torch.full((6,), 2.0), torch.full((V - 6,), -30.0)]))  # six equal tokens carry everything
    logits = torch.stack(rows).to(DEV)
    B = logits.shape[0]
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    checked = 0
    small = V < 10000   # the plain walk over a large vocabulary is slow: fewer draws there
    near = 1e-5 if small else 1e-6   # how close to a boundary a scaled coin may lie and still be compared
    for temp, tp in (((1.0, 0.9), (0.7, 0.5), (1.3, 0.95), (1.0, 0.999), (1.0, 0.05)) if small else ((0.7, 0.9), (1.0, 0.5))):
        probs = [P.temperature_probs(logits[b].double().cpu(), temp) for b in range(B)]
        for coin in ((0.0, 0.013, 0.2, 0.37, 0.5, 0.77, 0.93, 0.9999) if small else (0.0, 0.2, 0.5, 0.93)):
            ops.sample(logits, temp, tp, torch.full((B,), coin, device=DEV), out)
            got = out.tolist()
            for b in range(B):
                tok, margin = P.sample_topp(probs[b], tp, coin)
                assert got[b] in P.top_p_keep(probs[b], tp) or margin < near, (V, temp, tp, coin, b)
                if margin > near:
                    assert got[b] == tok, (V, temp, tp, coin, b, got[b], tok)
                    checked += 1
    assert checked > (150 if small else 25)


def test_repetition_penalty():
    from odin_infer_b200.csrc import ops
    from tests.plain import qwen3_plain as P
    logits = torch.tensor([[1.0, -1.0, 3.0, 0.5], [2.0, 2.0, -2.0, 0.0]], device=DEV)
    recent = torch.tensor([[0, 1, 1, -1], [2, 2, 2, 3]], dtype=torch.int32, device=DEV)
    ref = torch.stack([P.repetition_penalty(logits[b].cpu(), [t for t in recent[b].tolist() if t >= 0], 2.0) for b in range(2)])
    ops.repetition_penalty(logits, recent, 2.0)
    assert torch.equal(logits.cpu(), ref)


@pytest.mark.parametrize("geom", [(4, 2, 16), (6, 2, 32), (8, 8, 64), (32, 8, 128), (5, 1, 128), (3, 3, 256), (16, 2, 64)])
@pytest.mark.parametrize("n_split", [1, 3, 16])
def test_attention_decode_against_plain_kernel_and_reference(geom, n_split):
    """The split-key decode kernel: every sequence at its own length (1 .. several pages),
    scrambled pages, a padding row, all split counts; against a direct computation."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    lengths = [1, 64, 65, 200, 333]
    B = len(lengths)
    torch.manual_seed(n_q + hd + n_split)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    keys = [torch.randn(n, n_kv, hd, device=DEV).bfloat16() for n in lengths]
    vals = [torch.randn(n, n_kv, hd, device=DEV).bfloat16() for n in lengths]
    for s, n in enumerate(lengths):
        for p in range(n):
            page = int(bt[s, p // 64])
            k_cache[page, :, p % 64] = keys[s][p]
            v_cache[page, :, p % 64] = vals[s][p]
    # rows: the sequences in a shuffled order plus one padding row in the middle
    order = [3, 0, -1, 4, 1, 2]
    tok_seq = torch.tensor(order, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lengths[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    q = torch.randn(len(order), n_q * hd, device=DEV).bfloat16()
    out = torch.full((len(order), n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    scratch = torch.empty(ops.attention_decode_scratch(len(order), n_q, hd, n_split), device=DEV)
    ops.attention_decode(q, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0, scratch, n_split)
    plain = torch.full_like(out, 7.0)
    ops.attention_plain(q, plain, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0)
    assert torch.equal(out[2], torch.full_like(out[2], 7.0)), "a padding row must not be written"
    for r, s in enumerate(order):
        if s < 0:
            continue
        qs = q[r].double().view(n_q, hd).cpu()
        ref = torch.zeros(n_q, hd, dtype=torch.float64)
        for h in range(n_q):
            kh = h // (n_q // n_kv)
            sc = (keys[s][:, kh].double().cpu() @ qs[h]) / math.sqrt(hd)
            ref[h] = torch.softmax(sc, 0) @ vals[s][:, kh].double().cpu()
        close(out[r].view(n_q, hd), ref, 1e-2)
        close(out[r].float(), plain[r].float(), 1e-2)


@pytest.mark.parametrize("geom", [(32, 8, 128), (8, 8, 64), (12, 3, 128)])
@pytest.mark.parametrize("case", ["long", "many"])
def test_attention_decode_slots_used_again(geom, case):
    """More pages per CTA than the kernel has shared-memory slots, so that slots are used again:
    few CTAs (the deep ring) with long sequences, and more CTAs than SMs (the shallow ring).
    The far key that carries all the weight lies in a page that comes through a reused slot."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    torch.manual_seed(11 + hd)
    lengths = [1500, 777, 1101] if case == "long" else [600 + 13 * i for i in range(40)]
    B = len(lengths)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    q = 0.1 * torch.randn(B, n_q, hd, device=DEV)
    far_vals = []
    for s, n in enumerate(lengths):
        keys = 0.1 * torch.randn(n, n_kv, hd, device=DEV)
        vals = torch.randn(n, n_kv, hd, device=DEV)
        far = n - 1 - 64 * (s % 3) - 7          # in one of the last pages: slots 0.. have been used again by then
        keys[far] = 0.0
        keys[far, :, 0] = 40.0
        far_vals.append(vals[far, 0].bfloat16().float())
        pages = bt[s, : (n + 63) // 64].long()
        pad = pages.numel() * 64 - n
        kp = torch.cat([keys, torch.full((pad, n_kv, hd), float('nan'), device=DEV)]).view(-1, 64, n_kv, hd).permute(0, 2, 1, 3)
        vp = torch.cat([vals, torch.full((pad, n_kv, hd), float('nan'), device=DEV)]).view(-1, 64, n_kv, hd).permute(0, 2, 1, 3)
        k_cache[pages] = kp.bfloat16()
        v_cache[pages] = vp.bfloat16()
    q[:, :, 0] = 40.0 / math.sqrt(hd) * 2
    qf = q.reshape(B, n_q * hd).bfloat16()
    tok_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    tok_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    ref = torch.empty(B, n_q * hd, device=DEV, dtype=torch.bfloat16)
    ops.attention_plain(qf, ref, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0)
    for n_split in (1, 2):
        out = torch.zeros_like(ref)
        scratch = torch.empty(ops.attention_decode_scratch(B, n_q, hd, n_split), device=DEV)
        for _ in range(3):  # the race this guards against depended on timing
            ops.attention_decode(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0, scratch, n_split)
            close(out.float(), ref.float(), 1e-2)
        for s in range(B):
            close(out[s].float().view(n_q, hd)[0], far_vals[s], 2e-2)
    ops.attention_decode_check()


@pytest.mark.parametrize("geom", [(32, 8, 128), (8, 2, 64), (16, 1, 128), (6, 3, 64)])
@pytest.mark.parametrize("parts", [0, 1, 3])
def test_attention_decode_with_head_prep_equals_the_two_kernels(geom, parts):
    """Decode attention that prepares its own heads against head preparation followed by decode
    attention: the same results bit for bit, in the output and in the cache; sequences whose
    newest token opens a page, fills one, or lies in a page that comes through a reused slot;
    a padding row; one and several key splits.  parts 0: a bfloat16 projection output."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    lengths = [1, 64, 65, 128, 200, 641, 1000]
    B = len(lengths)
    torch.manual_seed(3 + hd + parts)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    for s, n in enumerate(lengths):  # everything but the newest token is in the cache already
        pages = bt[s, : (n + 63) // 64].long()
        k_cache[pages] = torch.randn(pages.numel(), n_kv, 64, hd, device=DEV).bfloat16()
        v_cache[pages] = torch.randn(pages.numel(), n_kv, 64, hd, device=DEV).bfloat16()
        last = int(pages[-1])
        k_cache[last, :, (n - 1) % 64:] = float("nan")   # the newest token's place and what lies behind it
        v_cache[last, :, (n - 1) % 64:] = float("nan")
    order = [3, 0, -1, 6, 1, 5, 2, 4]
    tok_seq = torch.tensor(order, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lengths[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    T, width = len(order), (n_q + 2 * n_kv) * hd
    if parts == 0:
        qkv = torch.randn(T, width, device=DEV).bfloat16()
    else:
        qkv = torch.randn(parts, T, width, device=DEV) / math.sqrt(parts)
    q_norm = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    k_norm = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    ang = torch.arange(1100, device=DEV, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV) / (hd // 2)))[None, :]
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    for n_split in (1, 3):
        ka, va, kb, vb = k_cache.clone(), v_cache.clone(), k_cache.clone(), v_cache.clone()
        scratch = torch.empty(ops.attention_decode_scratch(T, n_q, hd, n_split), device=DEV)
        q = ops.head_prep(qkv.clone(), n_q, n_kv, hd, q_norm, k_norm, 1e-6, cos, sin, hd, tok_pos, tok_seq, bt, ka, va,
                          q_out=torch.empty(T, n_q * hd, device=DEV, dtype=torch.bfloat16))
        ref = torch.full((T, n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
        ops.attention_decode(q, ref, n_q, n_kv, hd, ka, va, tok_pos, tok_seq, bt, 0, scratch, n_split)
        out = torch.full_like(ref, 7.0)
        assert ops.attention_decode_fused(qkv, out, n_q, n_kv, hd, q_norm, k_norm, 1e-6, cos, sin, hd, kb, vb,
                                          tok_pos, tok_seq, bt, 0, scratch, n_split)
        assert torch.equal(out, ref)
        for s, n in enumerate(lengths):  # the newest token's key and value, bit for bit
            page, row = int(bt[s, (n - 1) // 64]), (n - 1) % 64
            assert torch.equal(ka[page, :, row], kb[page, :, row]) and torch.equal(va[page, :, row], vb[page, :, row])
            assert not torch.isnan(kb[page, :, row].float()).any()
    ops.attention_decode_check()


@pytest.mark.parametrize("geom", [(32, 8, 128), (16, 8, 64), (8, 8, 128)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_of_more_items_than_ctas(geom, window):
    """Many more (sequence, kv head, split) items than CTAs fit on the GPU at once (980 to 4,900 for 296 places):
    sequences of 1 token to 11 pages in a shuffled order (items of one page, items whose last page is full or just
    begun, splits that find no page), padding rows, one key per sequence that carries all the weight; against the
    direct kernel; and a row's result is the same bits whatever else is in the batch (a few rows alone run with
    the deep ring of one CTA per SM)."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    g = n_q // n_kv
    torch.manual_seed(17 + hd + window)
    lengths = [1, 64, 65, 128, 129, 200, 641, 700] + [int(x) for x in torch.randint(1, 700, (112,))]
    B = len(lengths)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    far_vals = []
    for s, n in enumerate(lengths):
        keys = 0.1 * torch.randn(n, n_kv, hd, device=DEV)
        vals = torch.randn(n, n_kv, hd, device=DEV)
        lo = max(0, n - window) if window else 0
        far = lo + (s * 37) % (n - lo)           # a visible key, anywhere in the sequence
        keys[far] = 0.0
        keys[far, :, 0] = 40.0
        far_vals.append(vals[far].bfloat16().float())
        pages = bt[s, : (n + 63) // 64].long()
        pad = pages.numel() * 64 - n
        kp = torch.cat([keys, torch.full((pad, n_kv, hd), float('nan'), device=DEV)]).view(-1, 64, n_kv, hd).permute(0, 2, 1, 3)
        vp = torch.cat([vals, torch.full((pad, n_kv, hd), float('nan'), device=DEV)]).view(-1, 64, n_kv, hd).permute(0, 2, 1, 3)
        k_cache[pages] = kp.bfloat16()
        v_cache[pages] = vp.bfloat16()
    order = torch.randperm(B).tolist()
    order[5:5] = [-1]
    order[60:60] = [-1, -1]
    T = len(order)
    tok_seq = torch.tensor(order, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lengths[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    q = 0.1 * torch.randn(T, n_q, hd, device=DEV)
    q[:, :, 0] = 40.0 / math.sqrt(hd) * 2
    qf = q.reshape(T, n_q * hd).bfloat16()
    ref = torch.full((T, n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
    ops.attention_plain(qf, ref, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, window)
    few = [3, 4, 9, 10, 61, 62, 63]            # rows (some of them padding) run again as a small batch: one CTA per item
    for n_split in (1, 2, 5):
        out = torch.full_like(ref, 7.0)
        scratch = torch.empty(ops.attention_decode_scratch(T, n_q, hd, n_split), device=DEV)
        for _ in range(2):
            ops.attention_decode(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, window, scratch, n_split)
        ops.attention_decode_check()
        close(out.float(), ref.float(), 1e-2)
        for r, s in enumerate(order):
            if s < 0:
                assert torch.equal(out[r], torch.full_like(out[r], 7.0)), "a padding row must not be written"
            else:
                close(out[r].float().view(n_kv, g, hd)[:, 0], far_vals[s], 2e-2)
        sub = torch.full((len(few), n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
        ops.attention_decode(qf[few].contiguous(), sub, n_q, n_kv, hd, k_cache, v_cache, tok_pos[few].contiguous(),
                             tok_seq[few].contiguous(), bt, window, scratch, n_split)
        assert torch.equal(sub, out[few]), "a row's result depends on the rest of the batch"
    ops.attention_decode_check()


@pytest.mark.parametrize("geom", [(32, 8, 128), (16, 8, 64)])
@pytest.mark.parametrize("parts", [0, 3])
def test_attention_decode_of_more_items_than_ctas_with_head_prep(geom, parts):
    """The same many items with head preparation inside the kernel, against head preparation followed by decode
    attention: the same bits in the output and in the cache."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    torch.manual_seed(23 + hd + parts)
    lengths = [1, 64, 65, 128, 129, 200, 641, 700] + [int(x) for x in torch.randint(1, 700, (112,))]
    B = len(lengths)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    for s, n in enumerate(lengths):  # everything but the newest token is in the cache already
        pages = bt[s, : (n + 63) // 64].long()
        k_cache[pages] = torch.randn(pages.numel(), n_kv, 64, hd, device=DEV).bfloat16()
        v_cache[pages] = torch.randn(pages.numel(), n_kv, 64, hd, device=DEV).bfloat16()
        last = int(pages[-1])
        k_cache[last, :, (n - 1) % 64:] = float("nan")   # the newest token's place and what lies behind it
        v_cache[last, :, (n - 1) % 64:] = float("nan")
    order = torch.randperm(B).tolist()
    order[7:7] = [-1]
    tok_seq = torch.tensor(order, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lengths[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    T, width = len(order), (n_q + 2 * n_kv) * hd
    qkv = torch.randn(T, width, device=DEV).bfloat16() if parts == 0 else torch.randn(parts, T, width, device=DEV) / math.sqrt(parts)
    q_norm = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    k_norm = (1 + 0.1 * torch.randn(hd, device=DEV)).bfloat16()
    ang = torch.arange(800, device=DEV, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(hd // 2, device=DEV) / (hd // 2)))[None, :]
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    for n_split in (1, 3):
        ka, va, kb, vb = k_cache.clone(), v_cache.clone(), k_cache.clone(), v_cache.clone()
        scratch = torch.empty(ops.attention_decode_scratch(T, n_q, hd, n_split), device=DEV)
        q = ops.head_prep(qkv.clone(), n_q, n_kv, hd, q_norm, k_norm, 1e-6, cos, sin, hd, tok_pos, tok_seq, bt, ka, va,
                          q_out=torch.empty(T, n_q * hd, device=DEV, dtype=torch.bfloat16))
        ref = torch.full((T, n_q * hd), 7.0, device=DEV, dtype=torch.bfloat16)
        ops.attention_decode(q, ref, n_q, n_kv, hd, ka, va, tok_pos, tok_seq, bt, 0, scratch, n_split)
        out = torch.full_like(ref, 7.0)
        assert ops.attention_decode_fused(qkv, out, n_q, n_kv, hd, q_norm, k_norm, 1e-6, cos, sin, hd, kb, vb,
                                          tok_pos, tok_seq, bt, 0, scratch, n_split)
        assert not torch.isnan(out.float()).any()
        assert torch.equal(out, ref)
        for s, n in enumerate(lengths):  # the newest token's key and value, bit for bit
            page, row = int(bt[s, (n - 1) // 64]), (n - 1) % 64
            assert torch.equal(ka[page, :, row], kb[page, :, row]) and torch.equal(va[page, :, row], vb[page, :, row])
            assert not torch.isnan(kb[page, :, row].float()).any()
    ops.attention_decode_check()


@pytest.mark.parametrize("hd,n,far", [(64, 300, 67), (128, 9000, 70), (128, 9000, 8191), (128, 8300, 4096), (64, 8193, 8128)])
def test_attention_decode_window_and_far_key(hd, n, far):
    """One key among hundreds or thousands is made to dominate; whichever page, warp or key split it
    falls to, the output must be its value (block tables of up to 141 pages, up to 16 splits)."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv = 4, 2
    torch.manual_seed(5)
    k_cache, v_cache, bt = paged_cache(1, [n], n_kv, hd, torch.bfloat16)
    keys = 0.1 * torch.randn(n, n_kv, hd, device=DEV)
    vals = torch.randn(n, n_kv, hd, device=DEV)
    keys[far] = 0.0
    keys[far, :, 0] = 40.0
    q = 0.1 * torch.randn(1, n_q, hd, device=DEV)
    q[0, :, 0] = 40.0 / math.sqrt(hd) * 2
    for pg in range((n + 63) // 64):
        page, m = int(bt[0, pg]), min(64, n - pg * 64)
        k_cache[page, :, :m] = keys[pg * 64:pg * 64 + m].transpose(0, 1).bfloat16()
        v_cache[page, :, :m] = vals[pg * 64:pg * 64 + m].transpose(0, 1).bfloat16()
    tok_pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    tok_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    qf = q.reshape(1, n_q * hd).bfloat16()
    out = torch.empty(1, n_q * hd, device=DEV, dtype=torch.bfloat16)
    for n_split in (1, 4, 7, 16):
        scratch = torch.empty(ops.attention_decode_scratch(1, n_q, hd, n_split), device=DEV)
        ops.attention_decode(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0, scratch, n_split)
        close(out.float().view(n_q, hd)[0], vals[far, 0].bfloat16().float(), 2e-2)
        ops.attention_decode(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, n - 1 - far, scratch, n_split)
        assert (out.float().view(n_q, hd)[0] - vals[far, 0]).abs().max() > 0.1      # just outside the window
        ref = torch.empty_like(out)
        ops.attention_plain(qf, ref, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, n - 1 - far)
        close(out.float(), ref.float(), 1e-2)
        ops.attention_decode(qf, out, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, n - far, scratch, n_split)
        close(out.float().view(n_q, hd)[0], vals[far, 0].bfloat16().float(), 2e-2)  # just inside


@pytest.mark.parametrize("geom", [(4, 2, 64), (8, 8, 64), (4, 1, 128), (6, 2, 128), (32, 8, 128)])
@pytest.mark.parametrize("window", [0, 50])
def test_attention_prefill_against_plain_kernel_and_reference(geom, window):
    """The flash kernel: prompts of unequal lengths that start at 0 or continue from a
    non-zero position, pages scrambled, lengths around the tile and page sizes; unwritten
    cache slots hold NaN, which must never reach a result."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = geom
    # (already in the cache, new in this step)
    parts = [(0, 1), (0, 63), (0, 64), (0, 65), (0, 200), (70, 3), (64, 64), (5, 130)]
    lengths = [a + b for a, b in parts]
    B = len(parts)
    torch.manual_seed(n_q * 7 + hd + window)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    keys = [torch.randn(n, n_kv, hd, device=DEV).bfloat16() for n in lengths]
    vals = [torch.randn(n, n_kv, hd, device=DEV).bfloat16() for n in lengths]
    for s, n in enumerate(lengths):
        for pg in range((n + 63) // 64):
            page = int(bt[s, pg])
            a, b = pg * 64, min(n, pg * 64 + 64)
            k_cache[page, :, : b - a] = keys[s][a:b].transpose(0, 1)
            v_cache[page, :, : b - a] = vals[s][a:b].transpose(0, 1)
    T = sum(b for _, b in parts)
    q = torch.randn(T, n_q * hd, device=DEV).bfloat16()
    seq_start = torch.tensor([0] + list(np.cumsum([b for _, b in parts])), dtype=torch.int32, device=DEV)
    seq_len_after = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([a + i for a, b in parts for i in range(b)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([s for s, (a, b) in enumerate(parts) for _ in range(b)], dtype=torch.int32, device=DEV)
    out = torch.empty(T, n_q * hd, device=DEV, dtype=torch.bfloat16)
    ops.attention_prefill(q, out, B, max(b for _, b in parts), n_q, n_kv, hd, k_cache, v_cache, seq_start,
                          seq_len_after, bt, window)
    ops.attention_prefill_check()
    assert not torch.isnan(out.float()).any()
    plain = torch.empty_like(out)
    ops.attention_plain(q, plain, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, window)
    close(out.float(), plain.float(), 1e-2)
    r = 0
    for s, (a, b) in enumerate(parts):
        n = a + b
        qs = q[r:r + b].double().view(b, n_q, hd).cpu()
        pos = torch.arange(a, n)
        t = torch.arange(n)
        allowed = t[None, :] <= pos[:, None]
        if window:
            allowed &= t[None, :] > pos[:, None] - window
        for h in range(n_q):
            kh = h // (n_q // n_kv)
            sc = (qs[:, h] @ keys[s][:, kh].double().cpu().t()) / math.sqrt(hd)
            sc = sc.masked_fill(~allowed, float("-inf"))
            ref = torch.softmax(sc, -1) @ vals[s][:, kh].double().cpu()
            close(out[r:r + b].view(b, n_q, hd)[:, h], ref, 1e-2)
        r += b


def test_mma_probe_measures_every_pattern():
    """The measuring kernel behind `microbench mma-rate`: every pattern runs to its end (no wait runs out) and
    reports plausible cycle counts: an MMA of N 256 takes longer than one of N 64, and a group that is waited
    for takes longer than issuing it."""
    from odin_infer_b200.csrc import ops
    n64, _ = ops.mma_probe(0, 64, False, 0, 1, 256)
    n256, _ = ops.mma_probe(0, 256, False, 0, 1, 256)
    assert 8 < n64 < n256 < 2000
    ts, _ = ops.mma_probe(1, 128, True, 0, 2, 256)
    assert 8 < ts < 2000
    for pattern in (2, 3):
        page, _ = ops.mma_probe(pattern, 0, False, 1, 1, 32)
        assert 100 < page < 20000
    for pattern in (4, 5):
        whole, issue = ops.mma_probe(pattern, 0, False, 0, 1, 32)
        assert 0 < issue < whole < 20000
    with pytest.raises(ops.KernelError):
        ops.mma_probe(0, 72, False, 0, 1, 256)       # N is no multiple of 16


def test_attention_prefill_many_short_tiles_again_and_again():
    """Hundreds of tiles of one to five pages on persistent CTAs, launched thirty times: the barriers of a
    tile are armed again for the next one, and a page's loads may land before or after the MMA thread
    looks.  (A slot's barrier once ran two phases ahead of that thread in a tile of two pages, in a build
    with clock marks that slowed it; the ordinary build of that version passes this test, which guards
    the reuse of the barriers as such, not that race.)  Every launch must end without a wait that ran
    out and give the same bits; the first is compared with the plain kernel."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = 32, 8, 128
    torch.manual_seed(77)
    news = [1, 17, 63, 64, 65, 100, 127, 128, 129, 191, 192, 193, 255, 256, 257, 300] * 6
    olds = [(i * 37) % 130 if i % 3 == 0 else 0 for i in range(len(news))]
    parts = list(zip(olds, news))
    lengths = [a + b for a, b in parts]
    B = len(parts)
    k_cache, v_cache, bt = paged_cache(B, lengths, n_kv, hd, torch.bfloat16)
    for s, n in enumerate(lengths):
        for pg in range((n + 63) // 64):
            page = int(bt[s, pg])
            m = min(n, pg * 64 + 64) - pg * 64
            k_cache[page, :, :m] = torch.randn(n_kv, m, hd, device=DEV).bfloat16()
            v_cache[page, :, :m] = torch.randn(n_kv, m, hd, device=DEV).bfloat16()
    T = sum(news)
    q = torch.randn(T, n_q * hd, device=DEV).bfloat16()
    seq_start = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32, device=DEV)
    seq_len_after = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([a + i for a, b in parts for i in range(b)], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([s for s, (a, b) in enumerate(parts) for _ in range(b)], dtype=torch.int32, device=DEV)
    first = None
    for rep in range(30):
        out = torch.empty(T, n_q * hd, device=DEV, dtype=torch.bfloat16)
        ops.attention_prefill(q, out, B, max(news), n_q, n_kv, hd, k_cache, v_cache, seq_start, seq_len_after, bt, 0)
        ops.attention_prefill_check()
        if first is None:
            first = out
            assert not torch.isnan(out.float()).any()
            plain = torch.empty_like(out)
            ops.attention_plain(q, plain, n_q, n_kv, hd, k_cache, v_cache, tok_pos, tok_seq, bt, 0)
            close(out.float(), plain.float(), 1e-2)
        else:
            assert torch.equal(out, first), f"launch {rep} differs from the first"


@pytest.mark.parametrize("n,far", [(2048, 100), (8448, 100), (8448, 8191)])
def test_attention_prefill_long_prompt_far_key(n, far):
    """Thousands of tokens: one key of the prompt is made to dominate every later query."""
    from odin_infer_b200.csrc import ops
    n_q, n_kv, hd = 4, 2, 128
    torch.manual_seed(9)
    k_cache, v_cache, bt = paged_cache(1, [n], n_kv, hd, torch.bfloat16)
    keys = 0.05 * torch.randn(n, n_kv, hd, device=DEV)
    vals = torch.randn(n, n_kv, hd, device=DEV)
    keys[far] = 0.0
    keys[far, :, 5] = 30.0
    q = 0.05 * torch.randn(n, n_q, hd, device=DEV)
    q[:, :, 5] = 30.0 / math.sqrt(hd) * 3
    for pg in range(n // 64):
        page = int(bt[0, pg])
        k_cache[page] = keys[pg * 64:pg * 64 + 64].transpose(0, 1).bfloat16()
        v_cache[page] = vals[pg * 64:pg * 64 + 64].transpose(0, 1).bfloat16()
    out = torch.empty(n, n_q * hd, device=DEV, dtype=torch.bfloat16)
    seq_start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    seq_len_after = torch.tensor([n], dtype=torch.int32, device=DEV)
    ops.attention_prefill(q.reshape(n, -1).bfloat16(), out, 1, n, n_q, n_kv, hd, k_cache, v_cache, seq_start,
                          seq_len_after, bt, 0)
    ops.attention_prefill_check()
    got = out.float().view(n, n_q, hd)
    for t in (far, far + 1, min(far + 777, n - 2), n - 1):
        for h in range(n_q):
            close(got[t, h], vals[far, h // 2].bfloat16().float(), 2e-2)
    assert (got[far - 1, 0] - vals[far, 0]).abs().max() > 0.1   # causal: the key is not yet visible

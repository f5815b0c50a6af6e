"""Python bindings of the kernels: torch tensors in, raw pointers out.

Every function launches on torch's current CUDA stream (so a CUDA graph
capture records it), checks its arguments on the host, and raises on any
error code.  There is no fallback of any kind: a tensor that is not on a
CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build

PAGE = 64  # tokens per cache page

_DT = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise KernelError(f"unsupported element type {dt}; kernels take float32 and bfloat16") from None


def _ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError("kernel argument is not on a CUDA device (there is no CPU path)")
    return c_void_p(t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_ERRORS = {-1: "unsupported size or element type", -2: "bad argument", -3: "device wait ran out"}


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (kernels inside replayed CUDA graphs included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        msg = _ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {msg}")
    _launches += kernels


def _fn(group: str, name: str):
    """A launcher of the kernel libraries."""
    f = getattr(build.load(group), name)
    f.restype = c_int
    return f


# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[ids[t], :] as 32-bit floats; ids int32 [T]."""
    T, d = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == d
    assert table.is_contiguous() and out.is_contiguous()
    _check(_fn("elementwise", "odin_embed")(
        _ptr(table), c_int(dtype_code(table.dtype)), _ptr(ids), _ptr(out), c_int(T), c_int(d),
        c_int(table.shape[0]), _stream()), "embed")


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """x += sum of delta's leading splits (in place, 32-bit); out = RMSNorm(x) * weight.

    x: [n, d] float32.  delta: None, [n, d] or [splits, n, d].  rows: None, or
    int32 row numbers to gather (then x is left as it is).
    """
    d = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n_split, stride = 1, 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-1] == d
        if delta.dim() == 3:
            n_split, stride = delta.shape[0], delta.shape[1] * d
            assert delta.shape[1] == x.shape[0]
        else:
            assert delta.shape[0] == x.shape[0]
    n_rows = out.shape[0]
    if rows is None:
        assert n_rows == x.shape[0]
    else:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    assert weight.numel() == d
    _check(_fn("elementwise", "odin_add_rmsnorm")(
        _ptr(x), _ptr(delta), c_int(dtype_code(delta.dtype) if delta is not None else 0), c_int(n_split),
        c_longlong(stride), _ptr(weight), c_int(dtype_code(weight.dtype)), c_float(eps), _ptr(out),
        c_int(dtype_code(out.dtype)), _ptr(rows), c_int(n_rows), c_int(d), _stream()), "add_rmsnorm")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate) * up for gate_up = [T, 2I] (gate columns first), or for the sum of
    its leading parts when gate_up is [parts, T, 2I] (float32 partial sums of a split product)."""
    T, I = out.shape
    assert gate_up.is_contiguous() and out.is_contiguous() and tuple(gate_up.shape[-2:]) == (T, 2 * I)
    n_split, stride = (gate_up.shape[0], T * 2 * I) if gate_up.dim() == 3 else (1, 0)
    _check(_fn("elementwise", "odin_swiglu")(
        _ptr(gate_up), c_int(dtype_code(gate_up.dtype)), c_int(n_split), c_longlong(stride), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(T), c_int(I), _stream()), "swiglu")


def random_fill(out: torch.Tensor, key: int, mean: float, scale: float) -> None:
    """out.flatten()[i] = mean + scale * (centred sum of eight 16-bit uniforms of stream `key` at i): the
    device side of the counter-based random weights (weights/random_init.py has the host side)."""
    assert out.is_contiguous()
    _check(_fn("elementwise", "odin_random_fill")(
        _ptr(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)),
        c_float(mean), c_float(scale), _stream()), "random_fill")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _check(_fn("elementwise", "odin_cast")(
        _ptr(src), c_int(dtype_code(src.dtype)), _ptr(dst), c_int(dtype_code(dst.dtype)),
        c_longlong(src.numel()), _stream()), "cast")


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T on the CUDA cores with 32-bit accumulation."""
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(_fn("gemm_plain", "odin_gemm_plain")(
        _ptr(a), c_int(dtype_code(a.dtype)), _ptr(w), c_int(dtype_code(w.dtype)), _ptr(out),
        c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)),
        c_longlong(w.stride(0)), c_longlong(out.stride(0)), _stream()), "gemm_plain")


def gemm_tc_splits(K: int, n_split: int) -> int:
    """How many K parts `gemm_tc` really uses when asked for n_split."""
    f = build.load("gemm_tc").odin_gemm_tc_splits
    f.restype = c_int
    return int(f(c_int(K), c_int(n_split)))


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes and strides that the tensor-core kernel takes (TMA wants 16-byte rows)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
            and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, bn: int, n_split: int = 1,
            stages: int = 0, staged: int = 0) -> None:
    """out = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    mode 0: tokens on the 128-row side of the MMA, tiles of bn weight rows.
    mode 1: weight rows on the 128-row side, tiles of bn tokens (M <= bn is usual).
    n_split > 1: out is float32 [n_split, M, N]; slice s holds the partial sum of K part s.
    stages: length of the kernel's ring of shared-memory stages; 0: as many as fit, fewer to
    leave room on the SM for a CTA of the neighbouring kernel.
    staged (mode 1): K blocks of every CTA's first item whose weights are fetched into tensor memory
    while the kernel before this one still runs; changes no bit of the result.
    """
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and out.stride(-1) == 1
    if n_split > 1 or out.dim() == 3:
        assert out.dtype == torch.float32 and out.dim() == 3 and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_splits(K, n_split), "allocate gemm_tc_splits(K, n_split) slices"
        ldc, stride = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (M, N)
        ldc, stride = out.stride(0), 0
    _check(_fn("gemm_tc", "odin_gemm_tc")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(ldc), c_int(mode), c_int(bn), c_int(n_split),
        c_longlong(stride), c_int(stages), c_int(staged), _stream()), "gemm_tc")


def gemm_tc_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a Wg^T) * (a Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K]) in one tcgen05 kernel."""
    M, K = a.shape
    I = out.shape[1]
    if not gemm_tc_supported(a, w_gate_up):
        raise KernelError("gemm_tc_swiglu: operands must be bfloat16 with 16-byte aligned rows")
    assert w_gate_up.shape == (2 * I, K) and out.shape[0] == M and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc_swiglu")(
        _ptr(a), _ptr(w_gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)), _stream()),
        "gemm_tc_swiglu")


def gemm_tc2(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out = a[M, K] @ w[N, K]^T on pairs of SMs (tcgen05 cta_group::2, tiles of 256 x 256): for many tokens.
    accumulate: out (float32) += the product."""
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc2: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and tuple(out.shape) == (M, N) and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc2")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(out.stride(0)), c_int(1 if accumulate else 0),
        _stream()), "gemm_tc2")


def gemm_tc2_wide(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_split: int = 1) -> None:
    """out = a[M, K] @ w[N, K]^T for some hundred tokens on pairs of SMs, the weights on the wide side of the
    MMA and the tokens in tiles of 256 on its N side: out is [M, N], or float32 [n_split, M, N] partial sums of
    the K parts (as `gemm_tc`)."""
    M, K = a.shape
    N = w.shape[0]
    if not gemm_tc_supported(a, w):
        raise KernelError("gemm_tc2_wide: operands must be bfloat16 with 16-byte aligned rows (K and strides multiples of 8)")
    assert w.shape[1] == K and out.stride(-1) == 1
    if out.dim() == 3:
        assert out.dtype == torch.float32 and tuple(out.shape[1:]) == (M, N)
        assert out.shape[0] == gemm_tc_splits(K, n_split), "allocate gemm_tc_splits(K, n_split) slices"
        ldc, stride = out.stride(1), out.stride(0)
    else:
        assert tuple(out.shape) == (M, N) and n_split == 1
        ldc, stride = out.stride(0), 0
    _check(_fn("gemm_tc", "odin_gemm_tc2_wide")(
        _ptr(a), _ptr(w), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(N), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(ldc), c_int(n_split), c_longlong(stride),
        _stream()), "gemm_tc2_wide")


def gemm_tc2_swiglu_supported(inner: int) -> bool:
    return inner % 64 == 0


def gemm_tc2_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a Wg^T) * (a Wu^T) for w_gate_up = [Wg; Wu] ([2 I, K]) on pairs of SMs; I a multiple of 64."""
    M, K = a.shape
    I = out.shape[1]
    if not gemm_tc_supported(a, w_gate_up):
        raise KernelError("gemm_tc2_swiglu: operands must be bfloat16 with 16-byte aligned rows")
    assert w_gate_up.shape == (2 * I, K) and out.shape[0] == M and out.stride(1) == 1
    _check(_fn("gemm_tc", "odin_gemm_tc2_swiglu")(
        _ptr(a), _ptr(w_gate_up), _ptr(out), c_int(dtype_code(out.dtype)), c_int(M), c_int(I), c_int(K),
        c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)), _stream()),
        "gemm_tc2_swiglu")


def gemm_tc_check() -> None:
    """Raise if a tensor-core kernel gave up a bounded wait since the last check (synchronises)."""
    lib = build.load("gemm_tc")
    detail = (c_int * 8)()
    lib.odin_gemm_tc_error_detail.restype = c_int
    lib.odin_gemm_tc_error_detail(detail)
    f = lib.odin_gemm_tc_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("gemm_tc: a device-side wait ran out (pipeline stalled); results are invalid "
                          f"[wait, block, item, k block, slot, mode, tile, grid] = {list(detail)}")
    lib.odin_gemm_tc2_error.restype = c_int
    if lib.odin_gemm_tc2_error(detail) != 0:
        raise KernelError("gemm_tc2: a device-side wait ran out (pipeline stalled); results are invalid "
                          f"[wait, block, tile, k block, slot, 2, tile, grid] = {list(detail)}")


def head_prep(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, q_norm: torch.Tensor | None,
              k_norm: torch.Tensor | None, eps: float, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int,
              tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
              k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, write_kv: bool = True,
              q_out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-head RMSNorm and rotation of q and k, and the cache write of k and v.

    qkv: [T, (n_q + 2 n_kv) head_dim], or float32 partial sums [parts, T, ...] of a split
    product (added first).  q goes to q_out ([T, n_q head_dim], of the cache's type); without
    q_out it is written back into qkv (one part only).  Returns the tensor that holds q."""
    width = (n_q + 2 * n_kv) * head_dim
    if qkv.dim() == 3:
        n_split, T = qkv.shape[0], qkv.shape[1]
        assert qkv.is_contiguous() and qkv.shape[2] == width
        split_stride, row_stride = T * width, width
        assert q_out is not None, "partial sums need a separate q_out"
    else:
        n_split, T, split_stride, row_stride = 1, qkv.shape[0], 0, qkv.stride(0)
        assert qkv.stride(1) == 1 and qkv.shape[1] == width
    if q_out is None:
        q_out = qkv[:, : n_q * head_dim]
    assert q_out.stride(1) == 1 and tuple(q_out.shape) == (T, n_q * head_dim)
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32
    assert tok_pos.dtype == torch.int32 and tok_seq.dtype == torch.int32 and block_table.dtype == torch.int32
    has_norm = q_norm is not None
    if has_norm:
        assert k_norm is not None and q_norm.dtype == k_norm.dtype
        assert q_norm.numel() == head_dim and k_norm.numel() == head_dim
    if write_kv:
        assert k_cache is not None and v_cache is not None
        assert k_cache.dtype == q_out.dtype and v_cache.dtype == q_out.dtype
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim), "cache layout is [page][kv head][64][hd]"
    _check(_fn("head_prep", "odin_head_prep")(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(n_split), c_longlong(split_stride), _ptr(q_out),
        c_longlong(q_out.stride(0)), c_int(dtype_code(q_out.dtype)), c_int(T), c_int(n_q), c_int(n_kv),
        c_int(head_dim), c_longlong(row_stride), _ptr(q_norm), _ptr(k_norm),
        c_int(dtype_code(q_norm.dtype) if has_norm else 0), c_int(1 if has_norm else 0), c_float(eps),
        _ptr(cos), _ptr(sin), c_int(rotary_dim), c_int(cos.shape[0]), _ptr(tok_pos), _ptr(tok_seq),
        _ptr(block_table), c_int(block_table.stride(0)), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        c_int(1 if write_kv else 0), _stream()), "head_prep")
    return q_out


def attention_plain(q: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                    block_table: torch.Tensor, window: int = 0) -> None:
    """Causal attention of each token over its sequence's cache; q may be a strided view."""
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_cache.dtype
    assert q.shape[1] == n_q * head_dim and out.shape == (T, n_q * head_dim)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous()
    _check(_fn("attention_plain", "odin_attention_plain")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(dtype_code(q.dtype)),
        c_int(T), c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)), c_int(window),
        _stream()), "attention_plain")


def attention_decode_supported(head_dim: int) -> bool:
    return head_dim in (16, 32, 64, 128, 256)


def attention_decode_scratch(n_tokens: int, n_q: int, head_dim: int, n_split: int) -> int:
    """Floats of scratch that `attention_decode` needs."""
    return n_tokens * n_q * n_split * (head_dim + 2)


def attention_decode(q: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                     k_cache: torch.Tensor, v_cache: torch.Tensor, tok_pos: torch.Tensor, tok_seq: torch.Tensor,
                     block_table: torch.Tensor, window: int, scratch: torch.Tensor, n_split: int) -> None:
    """One query token per row over its sequence's bfloat16 cache, keys split n_split ways.

    The counters on which a launch's key splits meet are one array of the library: all
    decode-attention launches of a process must be ordered on the GPU (one stream, or events
    between streams); two that overlap would mix their arrivals."""
    B = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    assert q.shape[1] == n_q * head_dim and out.shape == (B, n_q * head_dim)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous()
    assert scratch.dtype == torch.float32 and scratch.numel() >= attention_decode_scratch(B, n_q, head_dim, n_split)
    _check(_fn("attention_decode", "odin_attention_decode")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv),
        c_int(head_dim), _ptr(k_cache), _ptr(v_cache), c_int(PAGE), c_int(k_cache.shape[0]), _ptr(tok_pos),
        _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)), c_int(window), _ptr(scratch), c_int(n_split),
        _stream()), "attention_decode", kernels=1 if head_dim in (64, 128) and n_q // n_kv <= 16 else 2)


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, n_q: int, n_kv: int, head_dim: int,
                           q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float, cos: torch.Tensor,
                           sin: torch.Tensor, rotary_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor, window: int,
                           scratch: torch.Tensor, n_split: int, write_kv: bool = True) -> bool:
    """`head_prep` and `attention_decode` in one kernel, for one token per sequence: qkv is the
    fused projection's output ([B, width] bfloat16, or float32 partial sums [parts, B, width]).
    Returns False, and launches nothing, where the tensor-core kernel does not apply; the
    caller then runs the two kernels."""
    width = (n_q + 2 * n_kv) * head_dim
    if qkv.dim() == 3:
        parts, B = qkv.shape[0], qkv.shape[1]
        if not (qkv.is_contiguous() and qkv.shape[2] == width and qkv.dtype == torch.float32):
            return False
        part_stride, row_stride = B * width, width
    else:
        parts, B, part_stride, row_stride = 1, qkv.shape[0], 0, qkv.stride(0)
        if not (qkv.stride(1) == 1 and qkv.shape[1] == width and qkv.dtype in (torch.bfloat16, torch.float32)):
            return False
    if not (out.dtype == k_cache.dtype == v_cache.dtype == torch.bfloat16 and out.stride(1) == 1
            and tuple(out.shape) == (B, n_q * head_dim) and k_cache.is_contiguous() and v_cache.is_contiguous()
            and tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and cos.dtype == sin.dtype == torch.float32):
        return False
    has_norm = q_norm is not None
    if has_norm and not (k_norm is not None and q_norm.dtype == k_norm.dtype and q_norm.numel() == head_dim
                         and k_norm.numel() == head_dim):
        return False
    assert scratch.dtype == torch.float32 and scratch.numel() >= attention_decode_scratch(B, n_q, head_dim, n_split)
    code = _fn("attention_decode", "odin_attention_decode_fused")(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(parts), c_longlong(part_stride), c_longlong(row_stride),
        _ptr(out), c_longlong(out.stride(0)), c_int(B), c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(q_norm),
        _ptr(k_norm), c_int(dtype_code(q_norm.dtype) if has_norm else 0), c_int(1 if has_norm else 0), c_float(eps),
        _ptr(cos), _ptr(sin), c_int(rotary_dim), c_int(cos.shape[0]), _ptr(k_cache), _ptr(v_cache), c_int(PAGE),
        c_int(k_cache.shape[0]), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table), c_int(block_table.stride(0)),
        c_int(window), _ptr(scratch), c_int(n_split), c_int(1 if write_kv else 0), _stream())
    if code == -1:  # unsupported: nothing was launched
        return False
    _check(code, "attention_decode_fused")
    return True


def attention_decode_check() -> None:
    f = build.load("attention_decode").odin_attention_decode_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("attention_decode: a device-side wait ran out; results are invalid")


def attention_prefill_supported(head_dim: int) -> bool:
    return head_dim in (64, 128)


def attention_prefill(q: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_q: int, n_kv: int,
                      head_dim: int, k_cache: torch.Tensor, v_cache: torch.Tensor, seq_start: torch.Tensor,
                      seq_len_after: torch.Tensor, block_table: torch.Tensor, window: int = 0) -> None:
    """Flash attention of each sequence's new tokens (rows seq_start[b]..seq_start[b+1] of q) over its
    bfloat16 cache, which already holds this step's keys and values: tcgen05.mma with accumulators in
    tensor memory."""
    T = q.shape[0]
    assert q.dtype == out.dtype == k_cache.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == n_q * head_dim and out.shape == (T, n_q * head_dim)
    assert tuple(k_cache.shape[1:]) == (n_kv, PAGE, head_dim) and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert seq_start.dtype == torch.int32 and seq_len_after.dtype == torch.int32 and block_table.dtype == torch.int32
    _check(_fn("attention_prefill", "odin_attention_prefill_tc")(
        _ptr(q), c_longlong(q.stride(0)), _ptr(out), c_longlong(out.stride(0)), c_int(n_seqs), c_int(max_new),
        c_int(n_q), c_int(n_kv), c_int(head_dim), _ptr(k_cache), _ptr(v_cache), c_int(k_cache.shape[0]),
        _ptr(seq_start), _ptr(seq_len_after), _ptr(block_table), c_int(block_table.stride(0)), c_int(window),
        _stream()), "attention_prefill")


def attention_prefill_check() -> None:
    detail = (c_int * 32)()
    build.load("attention_prefill").odin_attention_prefill_tc_error_detail(detail)
    for name in ("odin_attention_prefill_tc_error",):
        f = getattr(build.load("attention_prefill"), name)
        f.restype = c_int
        code = f()
        if code != 0:
            raise KernelError(f"attention_prefill ({name}): a device-side wait ran out or the kernel refused to run "
                              f"(code {code}); results are invalid; [wait, head, sequence, tile, iteration, pages, thread] = "
                              f"{list(detail)[:7]}; kinds that ran out (bit mask) {detail[7]:#x}, their last iterations + 1: {list(detail)[9:17]}")


def mma_probe(pattern: int, n: int = 64, b_mn: bool = False, commits: int = 0, per_sm: int = 1,
              iters: int = 4096) -> tuple[float, float]:
    """Cycles of the SM clock per MMA (patterns 0 and 1), per page / page pair (2 and 3) or per group of eight
    MMAs with its commit and wait (4 and 5) that the median CTA of the measuring kernel in mma_probe.cu took,
    and (4 and 5) the part of it until the eighth MMA was issued; per_sm CTAs share every SM's tensor core."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    grid = sms * per_sm
    cycles = torch.zeros(2 * grid, dtype=torch.int64, device="cuda:0")
    _check(_fn("mma_probe", "odin_mma_probe")(
        c_int(pattern), c_int(n), c_int(1 if b_mn else 0), c_int(commits), c_int(per_sm), c_int(iters),
        _ptr(cycles), _stream()), "mma_probe")
    torch.cuda.synchronize()
    f = build.load("mma_probe").odin_mma_probe_error
    f.restype = c_int
    if f() != 0:
        raise KernelError("mma_probe: a device-side wait ran out")
    whole, issue = cycles[:grid].sort().values, cycles[grid:].sort().values
    return float(whole[grid // 2].item()) / iters, float(issue[grid // 2].item()) / iters


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = index of the first maximum of logits[b, :] (float32)."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(_fn("sampling", "odin_argmax")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), _ptr(out), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_p: float, coins: torch.Tensor,
           out: torch.Tensor) -> None:
    """Temperature (and top-p) draw, one coin in [0, 1) per row."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert coins.dtype == torch.float32 and coins.numel() >= B and out.dtype == torch.int32
    _check(_fn("sampling", "odin_sample")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), c_float(temperature),
        c_float(top_p), _ptr(coins), _ptr(out), _stream()), "sample")


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: float) -> None:
    """In place on logits (a copy of the model's): recent is int32 [B, W], negative = empty."""
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert recent.dtype == torch.int32 and recent.is_contiguous() and recent.shape[0] == B
    _check(_fn("sampling", "odin_repetition_penalty")(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V), _ptr(recent),
        c_int(recent.shape[1]), c_float(penalty), _stream()), "repetition_penalty")

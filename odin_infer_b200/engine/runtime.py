"""The runtime a part sees: the element type of activations, the device, scratch
tensors, and the choice between kernel variants for matrix products and
attention.  Parts never choose a kernel themselves."""
from __future__ import annotations

import os

import torch

from ..csrc import ops
from ..parts.base import ResidualAdded


def choose_k_split(n_tiles: int, k_blocks: int, m: int, n_sms: int = 148, max_split: int = 16) -> int:
    """Into how many parts to cut K for a product of few tokens, so that the tiles fill
    the SMs in whole waves.  Cost of a choice, in units of one 64-wide K block of one
    tile: waves x (blocks per part + pipeline fill + the partial sums' traffic).
    The choice depends on the weight's shape alone, never on the tokens of the batch
    beyond their padded count, so a token's sums are cut the same way in every batch
    of the same bucket."""
    best, best_cost = 1, None
    for s in range(1, max_split + 1):
        per = (k_blocks + s - 1) // s
        if per < 4 and s > 1:
            break
        parts = (k_blocks + per - 1) // per
        waves = (n_tiles * parts + n_sms - 1) // n_sms
        cost = waves * (per + 4 + (m / 16.0 if parts > 1 else 0.0))
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = parts, cost
    return best


# Up to this many tokens a product keeps the weights on the wide side of the MMA and the tokens on
# its N side (one tile of tokens, K split to fill the SMs): with a few hundred tokens a product is still
# bound by the weights it streams, and tiles of 256 token rows would be too few to occupy the GPU (the o
# product of the 8B shape has 16 of them for 74 pairs of SMs).
WEIGHTS_WIDE_MAX_TOKENS = 256

# above that a product runs on pairs of SMs (tiles of 256 token rows)
PAIR_MIN_TOKENS = 257

# from this many tokens on the gate|up product carries the SwiGLU in its epilogue (see gated_linear)
SWIGLU_FUSED_FROM = int(os.environ.get("ODIN_SWIGLU_FUSED_FROM", "129"))

# up to this many tokens a product whose weight has few tiles still goes through the weights-wide
# kernel, in tiles of 256 tokens (see Runtime.linear)
WIDE_CHUNKS_MAX_TOKENS = int(os.environ.get("ODIN_WIDE_CHUNKS_MAX_TOKENS", "1024"))  # measured: faster up to there

# ring length of a product that shares the SM with a decode attention CTA (see Runtime.linear)
LIGHT_STAGES = int(os.environ.get("ODIN_GEMM_LIGHT_STAGES", "5"))

# K blocks of a few-token product's weights that wait in tensor memory while the kernel before it still runs
# (the kernel takes fewer where tensor or shared memory has no room); with the ring that is up to 400 KB an SM
STAGED_BLOCKS = int(os.environ.get("ODIN_GEMM_STAGED", "15"))


def context_class_of(longest: int, page: int = 64) -> int:
    """Contexts of one class launch the same kernels: the number of 8-page groups of the
    longest sequence."""
    return (max(1, (longest + page - 1) // page) + 7) // 8


def decode_key_splits(n_seqs: int, n_kv_heads: int, longest: int, page: int = 64, n_sms: int = 148,
                      ctas_per_sm: int = 2) -> int:
    """Into how many parts decode attention cuts a sequence's keys; the split that finishes last
    adds the partials up inside the same kernel.  Depends on the batch bucket and on the context
    class, never on which sequences are in the batch.

    Long contexts (more than 16 pages): the keys have to stream, so two splits per 8 pages as long
    as all CTAs together fit the GPU twice.

    Short contexts: the kernel is a chain of latencies, and what a choice costs is about, in
    microseconds on the 8B shape's decode step: 1.3 per round of pages (a CTA's four warps take a
    page each), 1.0 for the meeting of the splits if there is more than one, and 2.0 times the
    share of the CTAs that do not find an SM at once: a CTA that is there early, beside the
    projection's CTA on its SM, has its pages before the projection is done; one that comes later
    has not.  Of equal costs the larger number of splits wins.  (Measured, 520 to 580 tokens of
    context: 8 sequences: four splits 3.030 ms a step, three 3.044, one 3.056; 12 sequences: one
    split 3.134, two 3.155, three 3.173; 16 sequences: one 3.18, two 3.30; 4 sequences: four splits
    2.90, two 2.94.)"""
    forced = int(os.environ.get("ODIN_DECODE_SPLITS", "0"))
    if forced:
        return forced
    cls = context_class_of(longest, page)
    items = max(1, n_seqs * n_kv_heads)
    if cls > 2:
        room = max(1, (ctas_per_sm * n_sms) // items)
        return max(1, min(2 * cls, room, 16))  # a split that finds no page of its own writes an empty partial
    # one choice per class, whichever of its lengths comes first: for the class's shortest context (in the first
    # class: for half of its eight pages)
    pages = max(4, (cls - 1) * 8 + 1)
    room = max(1, (ctas_per_sm * n_sms) // items)  # never more CTAs than fit the GPU twice
    best, best_cost = 1, None
    for s in range(1, min(pages, room, 2 * cls) + 1):  # at most two splits per 8 pages
        per = (pages + s - 1) // s
        busy = (pages + per - 1) // per  # splits that find pages
        cost = 1.3 * ((per + 3) // 4) + (1.0 if s > 1 else 0.0) + 2.0 * max(0, items * busy - n_sms) / n_sms
        if best_cost is None or cost <= best_cost + 1e-9:
            best, best_cost = s, cost
    return best


class Runtime:
    def __init__(self, device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 148

    def kernel_groups(self) -> set[str]:
        """Kernel libraries the runtime itself may launch, beside those of the parts."""
        if self.dtype != torch.bfloat16:
            return set()
        return {"gemm_tc", "attention_decode", "attention_prefill"}

    def context_class(self, longest: int) -> int:
        """Contexts of one class launch the same kernels (see decode_key_splits)."""
        return context_class_of(longest)

    def run(self, model, batch):
        """Run one step of `model`; returns the logits at the wanted rows."""
        return model.forward(self, batch)

    def empty(self, *shape, dtype: torch.dtype | None = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    # ---- matrix product: out[M, N] = a[M, K] @ w[N, K]^T -----------------
    def linear(self, a, w: torch.Tensor, out_dtype: torch.dtype | None = None,
               may_split: bool = False, beside_attention: bool = False, add_to: torch.Tensor | None = None):
        """bfloat16 operands that TMA can read go to the tcgen05 kernel, everything else
        (the 32-bit path, odd widths, tensors stored in 32-bit) to the CUDA-core kernel.

        may_split: the caller's consumer adds partial sums, so a product of few tokens
        may come back as float32 [parts, M, N] (split along K to occupy every SM).

        beside_attention: the product comes right before or after attention; for few tokens
        it then keeps a shorter ring of stages, so that a CTA of the decode attention kernel
        fits on the SM beside it and can fetch its pages (or this product its weights) while
        the other still runs.

        add_to: the 32-bit residual stream [M, N] that the result is meant for; a product of many
        tokens then adds to it in its epilogue and returns `ResidualAdded()` instead of the update."""
        M, N, K = a.shape[0], w.shape[0], a.shape[1]
        out_dtype = out_dtype or self.dtype
        if M > 0 and ops.gemm_tc_supported(a, w):
            if M <= WEIGHTS_WIDE_MAX_TOKENS:
                bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
                n_split = choose_k_split((N + 127) // 128, (K + 63) // 64, M, self.n_sms) if may_split else 1
                n_split = ops.gemm_tc_splits(K, n_split)
                stages = LIGHT_STAGES if beside_attention else 0
                if M > 128:
                    # a few hundred tokens: on pairs of SMs, which halves what a CTA fetches per K block
                    n_tiles = (N + 255) // 256
                    n_split = ops.gemm_tc_splits(K, choose_k_split(n_tiles, (K + 63) // 64, M, self.n_sms // 2)
                                                 if may_split else 1)
                    out = self.empty(n_split, M, N, dtype=torch.float32) if n_split > 1 else self.empty(M, N, dtype=out_dtype)
                    ops.gemm_tc2_wide(a, w, out, n_split)
                    return out
                # tiles of 64 tokens and more: their token tiles would take the ring's shared memory (measured at 64
                # sequences: 4.82 to 5.28 ms a step with 5 to 12 blocks staged and the ring that much shorter, 4.80 without)
                staged = STAGED_BLOCKS if bn <= 32 else 0
                if n_split > 1:
                    out = self.empty(n_split, M, N, dtype=torch.float32)
                    ops.gemm_tc(a, w, out, 1, bn, n_split, stages, staged)
                    return out
                out = self.empty(M, N, dtype=out_dtype)
                ops.gemm_tc(a, w, out, 1, bn, 1, stages, staged)
                return out
        if (M > 0 and PAIR_MIN_TOKENS <= M <= WIDE_CHUNKS_MAX_TOKENS and may_split and ops.gemm_tc_supported(a, w)
                and (N + 255) // 256 < self.n_sms // 2):
            # Some hundred tokens and a weight of few 256-row tiles: tiles of 256 x 256 would leave most pairs
            # of SMs idle (the o product of the 8B shape: 16 tiles per 256 tokens for 74 pairs).  The tokens
            # go through the weights-wide kernel instead, in tiles of 256 tokens and K in parts; items that share
            # a weight tile run one after the other, so the second finds it in L2.
            items = ((N + 255) // 256) * ((M + 255) // 256)
            n_split = ops.gemm_tc_splits(K, choose_k_split(items, (K + 63) // 64, 256, self.n_sms // 2))
            out = self.empty(n_split, M, N, dtype=torch.float32) if n_split > 1 else self.empty(M, N, dtype=out_dtype)
            ops.gemm_tc2_wide(a, w, out, n_split)
            return out
        if M > 0 and ops.gemm_tc_supported(a, w):
            if (M >= PAIR_MIN_TOKENS and N > 128 and add_to is not None and out_dtype == torch.float32
                    and tuple(add_to.shape) == (M, N) and add_to.dtype == torch.float32 and add_to.stride(1) == 1):
                # many tokens: the product's epilogue adds to the residual stream in place
                ops.gemm_tc2(a, w, add_to, accumulate=True)
                return ResidualAdded()
            out = self.empty(M, N, dtype=out_dtype)
            if M >= PAIR_MIN_TOKENS and N > 128:
                ops.gemm_tc2(a, w, out)  # tiles of 256 x 256 on pairs of SMs
            else:
                ops.gemm_tc(a, w, out, 0, 256 if N > 128 else 128 if N > 64 else 64)
            return out
        out = self.empty(M, N, dtype=out_dtype)
        ops.gemm_plain(a, w, out)
        return out

    def gated_linear(self, a: torch.Tensor, w_gate_up: torch.Tensor, inner: int) -> torch.Tensor:
        """silu(a Wg^T) * (a Wu^T) for w_gate_up = [Wg; Wu]: one kernel with the SwiGLU in its
        epilogue for many bfloat16 tokens, else the product followed by the SwiGLU kernel
        (which also adds the partial sums of a split product)."""
        M = a.shape[0]
        act = self.empty(M, inner)
        # From 129 tokens on the pair kernel with the SwiGLU in its epilogue: the gate|up weight has tiles
        # enough for the pairs of SMs even beside one tile of 256 tokens, and no partial sums are written
        # (measured against the weights-wide kernel + SwiGLU kernel: 8 to 10 % of the step at 129 to 256 tokens).
        fused_from = SWIGLU_FUSED_FROM
        if M >= fused_from and ops.gemm_tc_supported(a, w_gate_up):
            if M > 128 and ops.gemm_tc2_swiglu_supported(inner):
                ops.gemm_tc2_swiglu(a, w_gate_up, act)
            else:
                ops.gemm_tc_swiglu(a, w_gate_up, act)
            return act
        ops.swiglu(self.linear(a, w_gate_up, may_split=True), act)
        return act

    # ---- attention over the cache ---------------------------------------
    def attention_with_head_prep(self, step, qkv, out, n_q, n_kv, head_dim, q_norm, k_norm, eps, cos, sin,
                                 rotary_dim, k_line, v_line, block_table, window, write_kv) -> bool:
        """One token per sequence in bfloat16: head preparation (per-head norm, rotation, the
        cache write) inside the attention kernel.  False where that kernel does not apply;
        the caller then prepares the heads and calls `attention`."""
        if os.environ.get("ODIN_FUSED_ATTENTION", "1") == "0":  # for comparisons
            return False
        if not (self.dtype == torch.bfloat16 and step.all_single and head_dim in (64, 128)
                and rotary_dim == head_dim and n_kv > 0 and n_q // n_kv <= 16 and write_kv):
            return False
        B = out.shape[0]
        n_split = decode_key_splits(B, n_kv, step.max_len_after, n_sms=self.n_sms)
        scratch = self.empty(ops.attention_decode_scratch(B, n_q, head_dim, n_split), dtype=torch.float32)
        return ops.attention_decode_fused(qkv, out, n_q, n_kv, head_dim, q_norm, k_norm, eps, cos, sin, rotary_dim,
                                          k_line, v_line, step.tok_pos, step.tok_seq, block_table, window, scratch,
                                          n_split, write_kv)

    def attention(self, step, q, out, n_q, n_kv, head_dim, k_line, v_line, block_table, window) -> None:
        """bfloat16: one token per sequence goes to the split-key kernel, prompts (and pieces
        of prompts) to the flash kernel.  The 32-bit path and head sizes that the fast
        kernels refuse go to the plain kernel."""
        if self.dtype == torch.bfloat16 and step.all_single and ops.attention_decode_supported(head_dim):
            B = q.shape[0]
            n_split = decode_key_splits(B, n_kv, step.max_len_after, n_sms=self.n_sms)
            scratch = self.empty(ops.attention_decode_scratch(B, n_q, head_dim, n_split), dtype=torch.float32)
            ops.attention_decode(q, out, n_q, n_kv, head_dim, k_line, v_line, step.tok_pos, step.tok_seq, block_table,
                                 window, scratch, n_split)
            return
        if self.dtype == torch.bfloat16 and not step.all_single and ops.attention_prefill_supported(head_dim):
            ops.attention_prefill(q, out, step.n_seq_cap, step.max_new, n_q, n_kv, head_dim, k_line, v_line,
                                  step.seq_start, step.seq_len_after, block_table, window)
            return
        ops.attention_plain(q, out, n_q, n_kv, head_dim, k_line, v_line, step.tok_pos, step.tok_seq, block_table,
                            window)

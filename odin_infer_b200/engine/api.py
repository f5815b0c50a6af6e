"""The engine: a loaded model, its cache, the step function and generation.

The public names follow the reference's library API (infer/engine.odin):
`Engine_Opts`, `engine_load`, `engine_forward`, `engine_config`,
`engine_destroy`.  Where the reference runs one token of one sequence per call
(infer/engine.odin:45), `Engine.step` runs a batch of sequences; the reference's
single-sequence call is kept as `engine_forward(e, token, pos)` on top of it.
"""
from __future__ import annotations

import dataclasses
import sys

import torch

from ..cache import CacheManager, PAGE, pages_for
from ..config import ModelConfig, load_config, lookup_architecture
from ..csrc import build as kernel_build
from ..sampling import PendingTokens, SamplingParams, sample_batch, sample_batch_async
from ..weights import load_weights, random_weights
from .graphs import DecodeGraphs
from .generate import GenerationResult, GenerationStats, generate
from .model import DecoderModel
from .runtime import Runtime
from .step import StepBatch, StepEntry, StepError

DEFAULT_MAX_CONTEXT = 4096  # infer/model.odin:10


@dataclasses.dataclass
class Engine_Opts:
    """max_ctx: cap on a sequence's length (infer/engine.odin:7-11; 0: the model's own
    limit, else min of both, infer/model.odin:220-223).  max_tokens: the most tokens
    that live sequences hold together, each rounded up to a page of 64; it sizes the
    cache (0: max_batch sequences of max_ctx).  dtype: "bfloat16" (the kernels and
    precisions of serving) or "float32" (everything in true 32-bit).  cuda_graphs: replay
    captured graphs for one-token-per-sequence steps (bfloat16 only).  run_ahead: generation
    launches a decode step before the host has read the tokens it continues from."""
    max_ctx: int = DEFAULT_MAX_CONTEXT
    max_tokens: int = 0
    max_batch: int = 8
    dtype: str = "bfloat16"
    device: str = "cuda:0"
    verbose: bool = True
    cuda_graphs: bool = True
    run_ahead: bool = True


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class Engine:
    def __init__(self, config: ModelConfig, opts: Engine_Opts, folder: str | None = None, seed: int | None = None):
        if opts.dtype not in _DTYPES:
            raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {opts.dtype!r}")
        if not torch.cuda.is_available():
            raise RuntimeError("odin_infer_b200 runs on a CUDA device (sm_100a) only; there is no CPU path")
        self.config = config
        self.opts = opts
        self.rt = Runtime(opts.device, _DTYPES[opts.dtype])
        self.run_ahead = opts.run_ahead
        torch.cuda.set_device(self.rt.device)
        spec = lookup_architecture(config.architecture).build_spec(config)
        self.spec = spec
        self.model = DecoderModel(spec)
        self.vocab_size = spec.vocab_size

        model_limit = spec.max_positions
        self.max_ctx = min(model_limit, opts.max_ctx) if (model_limit and opts.max_ctx > 0) else (opts.max_ctx or model_limit)
        if self.max_ctx <= 0:
            self.max_ctx = DEFAULT_MAX_CONTEXT
        self.max_batch = max(1, opts.max_batch)
        max_tokens = opts.max_tokens or self.max_batch * pages_for(self.max_ctx) * PAGE
        self.cache = CacheManager(max_tokens, self.max_ctx)
        self.max_ctx = self.cache.max_seq_len
        self.model.register_cache(self.cache)

        kernel_build.ensure_built(sorted(self.model.kernel_groups() | self.rt.kernel_groups()), verbose=opts.verbose)
        params = self.model.params()
        if folder is not None:
            tensors = load_weights(folder, params, self.rt.dtype, self.rt.device)
        else:
            tensors = random_weights(params, seed or 0, self.rt.dtype, self.rt.device)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in {id(t): t for t in tensors.values()}.values())
        self.model.bind(tensors, self.rt, self.max_ctx)
        del tensors

        itemsize = 4 if self.rt.dtype == torch.float32 else 2
        self.cache_bytes = 0
        for g in self.cache.groups.values():
            shape = g.storage_shape()
            k = torch.empty(shape, dtype=self.rt.dtype, device=self.rt.device)
            v = torch.empty(shape, dtype=self.rt.dtype, device=self.rt.device)
            g.attach_storage(k, v)
            self.cache_bytes += 2 * k.numel() * itemsize
        nstate = self.cache.state_bytes_per_slot
        self.cache.state = torch.zeros(self.cache.max_slots, nstate, dtype=torch.uint8, device=self.rt.device)
        self.cache.zero_state = (lambda slot: self.cache.state[slot].zero_()) if nstate else None
        # decode steps replay CUDA graphs in the serving precision; the 32-bit path stays eager
        self.last_step_h2d_bytes = 0
        self.graphs = None
        if opts.cuda_graphs and self.rt.dtype == torch.bfloat16:
            if self.model.graph_safe:
                self.graphs = DecodeGraphs(self.rt, self.model, self.cache)
            elif opts.verbose:
                print("odin_infer_b200: steps run eagerly, not as CUDA graphs: these parts do not declare graph_safe: "
                      + ", ".join(self.model.parts_not_graph_safe()), file=sys.stderr, flush=True)
        self.notes = self.model.notes(self.rt)
        if opts.verbose:
            print(self.summary(), file=sys.stderr, flush=True)
            for n in self.notes:
                print("odin_infer_b200: note: " + n, file=sys.stderr, flush=True)

    # ---- construction ------------------------------------------------------
    @classmethod
    def load(cls, folder: str, opts: Engine_Opts | None = None) -> "Engine":
        return cls(load_config(folder), opts or Engine_Opts(), folder=folder)

    @classmethod
    def random(cls, config: ModelConfig, seed: int, opts: Engine_Opts | None = None) -> "Engine":
        """Random weights generated on the device (nothing is written)."""
        return cls(config, opts or Engine_Opts(), seed=seed)

    def summary(self) -> str:
        """One line at load, as the reference prints (infer/model.odin:228-241)."""
        c = self.config
        return (f"odin_infer_b200: {c.architecture} {type(c).__name__} layers={len(self.spec.layers)} "
                f"width={self.spec.width} vocab={self.vocab_size} ctx={self.max_ctx} dtype={self.opts.dtype} "
                f"weights={self.weight_bytes / 2**30:.2f} GiB cache={self.cache_bytes / 2**20:.1f} MiB "
                f"({self.cache.n_pages} pages of {PAGE} tokens, {len(self.cache.groups)} group(s), "
                f"state {self.cache.state_bytes_per_slot} B/seq)")

    # ---- slots ------------------------------------------------------------
    def take_slot(self) -> int:
        return self.cache.take_slot()

    def give_back_slot(self, slot: int) -> None:
        self.cache.give_back_slot(slot)

    def fits(self, lengths: list[int]) -> bool:
        """Can sequences of these lengths be live together (beside what is live now)?"""
        need = sum(pages_for(n) for n in lengths)
        free = min((g.pool.n_free for g in self.cache.groups.values()), default=need)
        return need <= free and len(lengths) <= self.cache.n_free_slots

    def default_stop_token_ids(self) -> tuple[int, ...]:
        return tuple(self.spec.stop_token_ids)

    # ---- the step function ---------------------------------------------
    def step(self, entries: list[StepEntry], device_tokens=None) -> torch.Tensor | None:
        """Run the given tokens of every entry as one batch from the cache; returns the
        32-bit logits at the wanted places, [wanted, vocab], on the device, in the order
        of the entries and of their `want` lists (None when nothing is wanted).

        device_tokens = (tokens, src): every entry brings one token whose value is still on the
        device: entry b's is tokens[src[b]] (tokens[b] if src is None), tokens an int32 tensor as
        `sample_async` leaves it; the entries' own token values are placeholders then."""
        if not entries:
            return None
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.is_live(e.slot):
                raise StepError(f"slot {e.slot} is not held by a sequence")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a step must bring at least one token")
            for t in e.tokens:
                if not (0 <= t < self.vocab_size):  # infer/forward.odin:26-29
                    raise StepError(f"slot {e.slot}: token {t} is out of range (vocab {self.vocab_size})")
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {len(e.tokens)} token(s)")
        if device_tokens is not None and any(len(e.tokens) != 1 for e in entries):
            raise StepError("tokens from the device: one token per sequence")
        starts, grown = [], []
        try:
            for e in entries:
                starts.append(self.cache.extend(e.slot, len(e.tokens)))
                grown.append(e)
            logits = NotImplemented
            if self.graphs is not None and self.graphs.takes(entries):
                logits = self.graphs.run(entries, starts, device_tokens)
                self.last_step_h2d_bytes = self.graphs.last_h2d_bytes
            if logits is NotImplemented:
                batch = StepBatch(self.cache, entries, starts, self.rt.device)
                if device_tokens is not None:
                    batch.take_tokens(*device_tokens)
                logits = self.rt.run(self.model, batch)
                self.last_step_h2d_bytes = batch.h2d_bytes
        except Exception:
            # a step that did not run leaves lengths and pages as they were (what kernels may have
            # written lies beyond every sequence's length and is written again by the next step)
            for e, s in zip(grown, starts):
                self._shrink(e.slot, s)
            raise
        for e in entries:
            self.cache.after_step(e.slot)
        return logits

    def _shrink(self, slot: int, length: int) -> None:
        have, keep = pages_for(self.cache.lengths[slot]), pages_for(length)
        for g in self.cache.groups.values():
            pages = [int(p) for p in g.block_table[slot, keep:have] if p >= 0]
            g.pool.give_back(pages)
            g.block_table[slot, keep:have] = -1
        self.cache.lengths[slot] = length

    # ---- sampling and generation ----------------------------------------
    def sample(self, logits: torch.Tensor, samplers, params: SamplingParams) -> list[int]:
        return sample_batch(logits, samplers, params)

    def sample_async(self, logits: torch.Tensor, samplers, params: SamplingParams) -> PendingTokens:
        """Sampling that leaves the tokens on the device (for the next step's `device_tokens`) and
        copies them to the host in the background; `.tokens()` waits for that copy."""
        return sample_batch_async(logits, samplers, params)

    def generate(self, prompts, max_new_tokens: int = 256, temperature: float = 0.0, top_p: float = 1.0,
                 seed: int = 0, stop_token_ids=None, repetition_penalty: float = 1.0, include_stop_token: bool = False,
                 stats: GenerationStats | None = None) -> list[GenerationResult]:
        """prompts: lists of token ids.  Returns, in order, the generated tokens and why each ended."""
        params = SamplingParams(temperature=temperature, top_p=top_p, seed=seed, repetition_penalty=repetition_penalty)
        return generate(self, [list(map(int, p)) for p in prompts], max_new_tokens, params, stop_token_ids,
                        include_stop_token, stats)

    def destroy(self) -> None:
        for g in self.cache.groups.values():
            g.k = g.v = None
        self.cache.state = None
        if self.graphs is not None:
            self.graphs.clear()
        self.model = None
        torch.cuda.empty_cache()


# ---- the reference's procedural API (infer/engine.odin:18-60) -----------------
def engine_load(path: str, opts: Engine_Opts | None = None) -> Engine:
    """infer/engine.odin:18-34.  Raises instead of exiting the process."""
    return Engine.load(path, opts)


def engine_config(e: Engine) -> ModelConfig:
    """infer/engine.odin:54-56."""
    return e.config


def engine_forward(e: Engine, token: int, pos: int) -> torch.Tensor:
    """One token of one sequence at position `pos`; returns its 32-bit logits [vocab]
    (infer/engine.odin:45-52).  The engine keeps one slot for this call; pos 0 starts the
    sequence afresh, any other pos must be the next position."""
    slot = getattr(e, "_single_slot", None)
    if pos == 0:
        if slot is not None:
            e.give_back_slot(slot)
        slot = e._single_slot = e.take_slot()
    if slot is None or e.cache.lengths[slot] != pos:
        have = None if slot is None else e.cache.lengths[slot]
        raise StepError(f"engine_forward: pos={pos} is not the next position (the sequence holds {have} tokens)")
    if pos >= e.max_ctx:  # infer/forward.odin:22-25
        raise StepError(f"engine_forward: pos={pos} out of range (seq_len={e.max_ctx})")
    return e.step([StepEntry(slot, [int(token)], [0])])[0]


def engine_destroy(e: Engine) -> None:
    """infer/engine.odin:36-43."""
    e.destroy()

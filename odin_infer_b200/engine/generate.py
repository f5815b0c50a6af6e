"""The generation loop: requests in, token lists out.

Requests are taken in order into batches that start together: the prompts of a
batch run in one step (unequal lengths, no padding), then every live sequence
advances by one token per step.  A sequence ends at a stop token (not emitted,
not fed back: serve_harness/serve.odin:514-515 checks EOS before emitting), after
`max_new_tokens`, or when its length reaches the context limit (:521-522,
finish reason "length"); it then leaves the batch, which goes on smaller.  When
a batch is done its slots are given back and the next batch takes them.

With an engine whose sampling can leave the tokens on the device (`sample_async`,
and `step(..., device_tokens=...)`), the loop runs one step ahead of the host: it
launches the next decode step on the tokens that are still on the device and reads
the previous step's tokens while that step runs, so the host's share of a step
hides behind the device's.  Who ends by length is known before the token is, and
is left out of the step ahead; a sequence whose token turns out to be a stop token
has run one step for nothing.  The tokens and reasons that come out are the same.

The loop is written against a small interface (`take_slot`, `give_back_slot`,
`step`, `sample`, `max_batch`, `max_ctx`, `fits`; optionally `sample_async`), so
its decisions can be tested without a GPU.
"""
from __future__ import annotations

import dataclasses
import time

from ..sampling import SamplingParams, SequenceSampler
from .step import StepEntry


@dataclasses.dataclass
class GenerationResult:
    tokens: list[int]
    finish_reason: str            # "stop" or "length"
    prompt_tokens: int = 0


@dataclasses.dataclass
class GenerationStats:
    """TTFT and decode rate as the reference reports them (serve_harness/serve.odin:527-532:
    the rate excludes the prompt step)."""
    ttft_s: float = 0.0
    decode_s: float = 0.0
    decode_tokens: int = 0
    prefill_tokens: int = 0
    n_batches: int = 0
    n_steps: int = 0

    @property
    def decode_tokens_per_s(self) -> float:
        return self.decode_tokens / self.decode_s if self.decode_s > 0 else 0.0


@dataclasses.dataclass
class _Live:
    number: int
    slot: int
    prompt: list[int]
    sampler: SequenceSampler
    out: list[int] = dataclasses.field(default_factory=list)
    finish: str | None = None

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.out)


def plan_batches(prompt_lengths: list[int], max_new_tokens: int, max_batch: int, fits) -> list[list[int]]:
    """Request numbers grouped, in order, into batches.  `fits(lengths)` says whether
    sequences that may grow to these lengths can be live together."""
    batches: list[list[int]] = []
    cur: list[int] = []
    for i, n in enumerate(prompt_lengths):
        trial = cur + [i]
        if cur and (len(trial) > max_batch or not fits([prompt_lengths[j] + max_new_tokens for j in trial])):
            batches.append(cur)
            cur = [i]
        else:
            cur = trial
    if cur:
        batches.append(cur)
    return batches


def generate(engine, prompts: list[list[int]], max_new_tokens: int = 256, params: SamplingParams | None = None,
             stop_token_ids=None, include_stop_token: bool = False, stats: GenerationStats | None = None
             ) -> list[GenerationResult]:
    params = params or SamplingParams()
    stops = set(engine.default_stop_token_ids() if stop_token_ids is None else stop_token_ids)
    stats = stats if stats is not None else GenerationStats()
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i}: empty prompt")
        if len(p) >= engine.max_ctx:
            raise ValueError(f"request {i}: a prompt of {len(p)} tokens leaves no room under the context limit "
                             f"of {engine.max_ctx}")
    results: list[GenerationResult | None] = [None] * len(prompts)
    if max_new_tokens <= 0:
        return [GenerationResult([], "length", len(p)) for p in prompts]
    t_begin = time.perf_counter()
    first_token_seen = False
    # an engine that can sample without handing the tokens to the host first runs one step ahead;
    # the repetition penalty needs every token on the host before the next one is drawn
    ahead = (hasattr(engine, "sample_async") and getattr(engine, "run_ahead", True)
             and params.repetition_penalty == 1.0)
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, engine.max_batch,
                              lambda lens: engine.fits([min(n, engine.max_ctx) for n in lens])):
        stats.n_batches += 1
        live = [_Live(i, engine.take_slot(), prompts[i], SequenceSampler(params, i, prompts[i])) for i in batch]
        try:
            # the prompts, in one step; logits at each prompt's last place
            logits = engine.step([StepEntry(s.slot, s.prompt, [len(s.prompt) - 1]) for s in live])
            stats.n_steps += 1
            stats.prefill_tokens += sum(len(s.prompt) for s in live)
            t_decode0 = None

            def take(tokens_of: list[_Live], tokens: list[int]) -> None:
                """The sampled tokens of these sequences: who goes on, who ends, and why."""
                nonlocal first_token_seen, t_decode0
                if not first_token_seen:
                    first_token_seen = True
                    stats.ttft_s = time.perf_counter() - t_begin
                if t_decode0 is None:
                    t_decode0 = time.perf_counter()
                else:
                    stats.decode_tokens += sum(1 for s in tokens_of if s.finish is None)
                for s, tok in zip(tokens_of, tokens):
                    if s.finish is not None:  # ended a step ago; this token was computed for nothing
                        continue
                    if tok in stops:
                        if include_stop_token:
                            s.out.append(tok)
                        s.finish = "stop"
                        continue
                    s.out.append(tok)
                    if len(s.out) >= max_new_tokens or s.length >= engine.max_ctx:
                        s.finish = "length"
                for s in tokens_of:
                    if s.finish is not None and s.slot >= 0:
                        results[s.number] = GenerationResult(s.out, s.finish, len(s.prompt))
                        engine.give_back_slot(s.slot)
                        s.slot = -1

            if ahead:
                # One step ahead: the next step is launched with its input tokens still on the device,
                # before the host has read them; the host reads a step's tokens while the device runs
                # the next one.  A sequence whose token turns out to be a stop token has then run one
                # step for nothing (its row is ignored; its slot goes back as usual: what is launched
                # later runs later).  Sequences that end by length are known beforehand and left out.
                order = list(live)  # the sequences whose tokens `pending` holds, row by row
                pending = engine.sample_async(logits, [s.sampler for s in order], params)
                # the batch's first tokens go out before anything else is launched (whatever the first
                # decode step has to set up must not stand between a request and its first token)
                take(order, pending.tokens())
                taken = True
                while True:
                    if taken:
                        go_on = [s for s in order if s.finish is None]
                    else:
                        go_on = [s for s in order if s.finish is None and len(s.out) + 1 < max_new_tokens
                                 and s.length + 1 < engine.max_ctx]
                    pending_next = None
                    if go_on:
                        src = None if len(go_on) == len(order) else [order.index(s) for s in go_on]
                        logits = engine.step([StepEntry(s.slot, [0], [0]) for s in go_on],
                                             device_tokens=(pending.device_tokens, src))
                        stats.n_steps += 1
                        pending_next = engine.sample_async(logits, [s.sampler for s in go_on], params)
                    if not taken:
                        take(order, pending.tokens())
                    taken = False
                    live = [s for s in live if s.finish is None]
                    if not live or pending_next is None:
                        break
                    order, pending = go_on, pending_next
            else:
                while True:
                    tokens = engine.sample(logits, [s.sampler for s in live], params)
                    take(live, tokens)
                    live = [s for s in live if s.finish is None]
                    if not live:
                        break
                    logits = engine.step([StepEntry(s.slot, [s.out[-1]], [0]) for s in live])
                    stats.n_steps += 1
            stats.decode_s += time.perf_counter() - t_decode0
        finally:
            for s in live:
                if s.slot >= 0:
                    engine.give_back_slot(s.slot)
    return results  # type: ignore[return-value]

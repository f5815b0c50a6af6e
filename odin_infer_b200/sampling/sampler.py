"""Choosing the next token of every sequence of a batch.

Order of operations as in the reference's `sample` (sampler/sampler.odin:141-199):
repetition penalty, then argmax if the temperature is 0, else logits / T, softmax,
one coin per token, and a walk of the cumulative sum (all tokens, or the top-p set
when 0 < top_p < 1).  The arithmetic over the vocabulary runs in CUDA kernels
(csrc/sampling.cu); the host keeps the random streams and the windows of recent
tokens.

Random numbers: the reference's xorshift64* (sampler/sampler.odin:68-77: shifts
12, 25, 27, multiplier 0x2545F4914F6CDD1D, high 32 bits; float = (u32 >> 8) / 2^24).
Every sequence has a stream of its own, seeded from (seed, its number among the
requests), so what a sequence draws does not depend on who shares its batch.  The
reference's seed 0 is a fixed point of xorshift (every coin is 0); here the seed
is mixed first, so 0 is a seed like any other.
"""
from __future__ import annotations

import dataclasses

_MASK = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


class XorShift64Star:
    """sampler/sampler.odin:68-77."""

    def __init__(self, state: int):
        self.state = state & _MASK

    def random_u32(self) -> int:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK
        s ^= s >> 27
        self.state = s
        return ((s * 0x2545F4914F6CDD1D) & _MASK) >> 32

    def random_f32(self) -> float:
        return (self.random_u32() >> 8) / 16777216.0


def stream_for(seed: int, sequence_number: int) -> XorShift64Star:
    s = splitmix64(splitmix64(seed & _MASK) ^ (sequence_number & _MASK))
    return XorShift64Star(s or 0x9E3779B97F4A7C15)


@dataclasses.dataclass
class SamplingParams:
    """temperature 0: greedy.  top_p <= 0 or >= 1: off.  repetition_penalty 1: off
    (values below 1 are raised to 1, sampler/sampler.odin:43); it looks at the last
    `penalty_window` tokens of prompt and output (64 in the reference, :50)."""
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    repetition_penalty: float = 1.0
    penalty_window: int = 64

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
        if self.repetition_penalty < 1.0:
            self.repetition_penalty = 1.0


class SequenceSampler:
    """Host-side sampling state of one sequence: its random stream and recent tokens."""

    def __init__(self, params: SamplingParams, sequence_number: int, prompt: list[int]):
        self.params = params
        self.rng = stream_for(params.seed, sequence_number)
        self.recent: list[int] = []
        if params.repetition_penalty != 1.0:
            self.recent = list(prompt[-params.penalty_window:])

    def coin(self) -> float:
        return self.rng.random_f32()

    def record(self, token: int) -> None:
        if self.params.repetition_penalty != 1.0:
            self.recent.append(token)
            if len(self.recent) > self.params.penalty_window:
                del self.recent[0]


def sample_batch(logits, samplers: list[SequenceSampler], params: SamplingParams) -> list[int]:
    """logits: float32 [B, V] on the device, row b for samplers[b].  Returns B token ids.
    One device-to-host copy of B integers; the logits are left as they are."""
    import torch
    from ..csrc import ops

    B = logits.shape[0]
    assert B == len(samplers)
    dev = logits.device
    if params.repetition_penalty != 1.0:
        W = params.penalty_window
        recent = [(s.recent + [-1] * W)[:W] for s in samplers]
        logits = logits.clone()
        ops.repetition_penalty(logits, torch.tensor(recent, dtype=torch.int32).to(dev), params.repetition_penalty)
    out = torch.empty(B, dtype=torch.int32, device=dev)
    if params.temperature == 0.0:
        ops.argmax(logits, out)
    else:
        coins = torch.tensor([s.coin() for s in samplers], dtype=torch.float32).to(dev)
        ops.sample(logits, params.temperature, params.top_p, coins, out)
    tokens = out.cpu().tolist()
    for s, t in zip(samplers, tokens):
        s.record(t)
    return tokens


class PendingTokens:
    """Sampled tokens that are on the device (`device_tokens`, int32 [B]) and on their way to the
    host; `tokens()` waits for the copy."""

    def __init__(self, device_tokens):
        import torch
        self.device_tokens = device_tokens
        self._host = torch.empty(device_tokens.shape, dtype=device_tokens.dtype, pin_memory=device_tokens.is_cuda)
        self._host.copy_(device_tokens, non_blocking=True)
        self._event = None
        if device_tokens.is_cuda:
            self._event = torch.cuda.Event()
            self._event.record()

    def tokens(self) -> list[int]:
        if self._event is not None:
            self._event.synchronize()
        return self._host.tolist()


def sample_batch_async(logits, samplers: list[SequenceSampler], params: SamplingParams) -> PendingTokens:
    """`sample_batch` without waiting for the tokens: the same kernels and coins; the host sees the
    tokens when it asks for them.  Not with a repetition penalty, which needs each token on the host
    before the next one is drawn."""
    import torch
    from ..csrc import ops

    if params.repetition_penalty != 1.0:
        raise ValueError("sampling ahead of the host cannot apply a repetition penalty")
    B = logits.shape[0]
    assert B == len(samplers)
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    if params.temperature == 0.0:
        ops.argmax(logits, out)
    else:
        coins = torch.tensor([s.coin() for s in samplers], dtype=torch.float32).to(logits.device, non_blocking=True)
        ops.sample(logits, params.temperature, params.top_p, coins, out)
    return PendingTokens(out)

"""Sampling: greedy, temperature, top-p, repetition penalty."""
from .sampler import (PendingTokens, SamplingParams, SequenceSampler, XorShift64Star, sample_batch,
                      sample_batch_async, splitmix64, stream_for)

__all__ = ["PendingTokens", "SamplingParams", "SequenceSampler", "XorShift64Star", "sample_batch", "sample_batch_async",
           "splitmix64", "stream_for"]

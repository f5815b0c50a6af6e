"""Sampling: greedy, temperature, top-p, repetition penalty."""
from .sampler import SamplingParams, SequenceSampler, XorShift64Star, sample_batch, splitmix64, stream_for

__all__ = ["SamplingParams", "SequenceSampler", "XorShift64Star", "sample_batch", "splitmix64", "stream_for"]

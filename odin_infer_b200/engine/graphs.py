"""CUDA graphs of the decode step.

A step in which every sequence brings one token launches a few hundred small
kernels; at small batches the launches cost more than the kernels.  Such steps
are captured once per batch-size bucket and replayed: the step's integer tables
live in fixed device buffers that are refilled before every replay, padding rows
(sequence -1) make up the difference to the bucket size and change no result.

Only a model whose parts all say `graph_safe` is captured (the engine asks before it
builds this object).  A step that finds no graph yet runs eagerly, and that run IS the
step: the capture that follows records the same launches for later steps without
executing them, so nothing (keys, values, a mixer's fixed-size state) is applied twice.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .step import StepBatch, StepEntry

BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)

# Short prompts are launch-bound too when they run eagerly (a few hundred launches of ~25 us of host
# time each: 8 ms for what the device does in 3): steps of a few sequences with up to 1,024 tokens in
# all are captured as well, per bucket of their token count and of their number of sequences, padded
# with rows of sequence -1 and with empty sequences.
PROMPT_BUCKETS = (32, 64, 128, 192, 256, 384, 512, 768, 1024)
PROMPT_SEQ_BUCKETS = (1, 2, 4, 8, 16)


def bucket_for(n: int) -> int | None:
    for b in BUCKETS:
        if n <= b:
            return b
    return None


class DecodeGraphs:
    def __init__(self, rt, model, cache):
        self.rt, self.model, self.cache = rt, model, cache
        self._graphs: dict[tuple, tuple] = {}
        self.last_h2d_bytes = 0

    def takes(self, entries: list[StepEntry]) -> bool:
        """Is this a step that `run` may replay a graph for?"""
        if all(len(e.tokens) == 1 for e in entries):
            return True
        return (len(entries) <= PROMPT_SEQ_BUCKETS[-1] and sum(len(e.tokens) for e in entries) <= PROMPT_BUCKETS[-1]
                and any(e.want for e in entries))

    def _run_prompt(self, entries: list[StepEntry], starts: list[int]) -> torch.Tensor | None:
        """A few sequences' tokens (prompts or pieces of them) in a bucket of rows and of sequences."""
        n = sum(len(e.tokens) for e in entries)
        rows = next(b for b in PROMPT_BUCKETS if n <= b)
        seqs = next(b for b in PROMPT_SEQ_BUCKETS if len(entries) <= b)
        key = ("prompt", rows, seqs, sum(len(e.want) for e in entries))
        hit = self._graphs.get(key)
        if hit is None:
            batch = StepBatch(self.cache, entries, starts, self.rt.device, pad_rows_to=rows, pad_seqs_to=seqs)
            return self._first_run(key, batch)
        graph, batch, logits, n_kernels = hit
        batch.fill(entries, starts)
        graph.replay()
        ops.add_launches(n_kernels)
        self.last_h2d_bytes = batch.h2d_bytes
        return logits

    def _first_run(self, key, batch: StepBatch, device_tokens=None) -> torch.Tensor | None:
        """The step itself, eagerly (first-use set-up of the kernels - function attributes, tensor
        maps, error flags, the allocator's pools - must not fall into a capture), then the capture
        of the same launches for the steps to come.  Returns the eager run's logits."""
        if device_tokens is not None:
            batch.take_tokens(*device_tokens)
        logits = self.rt.run(self.model, batch)
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = ops.launch_count()
        with torch.cuda.graph(graph):
            captured = self.rt.run(self.model, batch)
        n_kernels = ops.launch_count() - n0
        ops.add_launches(-n_kernels)          # recorded, not launched
        self._graphs[key] = (graph, batch, captured, n_kernels)
        self.last_h2d_bytes = batch.h2d_bytes
        return logits

    def run(self, entries: list[StepEntry], starts: list[int], device_tokens=None) -> torch.Tensor | None:
        """Logits [wanted, vocab] of a one-token-per-sequence step (or of one sequence's short
        prompt), or NotImplemented if the batch is larger than the largest bucket."""
        if any(len(e.tokens) > 1 for e in entries):
            return self._run_prompt(entries, starts)
        bucket = bucket_for(len(entries))
        if bucket is None:
            return NotImplemented
        # kernels whose launch shape follows the longest context (decode attention's key splits)
        # make a graph valid for a class of context lengths only: the class is part of the key
        longest = max(s + 1 for s in starts)
        bucket = (bucket, self.rt.context_class(longest))
        hit = self._graphs.get(bucket)
        if hit is None:
            batch = StepBatch(self.cache, entries, starts, self.rt.device, pad_rows_to=bucket[0], pad_seqs_to=bucket[0],
                              all_rows_wanted=True)
            logits = self._first_run(bucket, batch, device_tokens)
        else:
            graph, batch, logits, n_kernels = hit
            batch.fill(entries, starts)
            if device_tokens is not None:  # the tokens come from the device: into the tables after their copy
                batch.take_tokens(*device_tokens)
            graph.replay()
            ops.add_launches(n_kernels)
            self.last_h2d_bytes = batch.h2d_bytes
        rows = batch.wanted_rows
        if not rows:
            return None
        if rows == list(range(len(rows))):
            return logits[:len(rows)]
        return logits[torch.tensor(rows, device=logits.device)]

    def clear(self) -> None:
        self._graphs.clear()

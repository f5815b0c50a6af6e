"""A running model put together from a ModelSpec: embedding, blocks in schedule
order, final norm, head.  Architecture-independent."""
from __future__ import annotations

import torch

from ..parts.base import ParamSpec, build_part
from ..parts.spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.position_encodings = {n: build_part("position_encoding", s) for n, s in spec.position_encodings.items()}
        self.layers = [build_part("block", s) for s in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"the schedule names layer {e.layer}; there are {len(self.layers)}")
        for blk in self.layers:
            name = getattr(blk.mixer, "pe_name", None)
            if name is not None:
                if name not in self.position_encodings:
                    raise ValueError(f"a mixer asks for position encoding '{name}', which the model does not define")
                blk.mixer.pe = self.position_encodings[name]

    def _all_parts(self):
        return [self.embedding, *self.position_encodings.values(), *self.layers, self.final_norm, self.head]

    def params(self) -> list[ParamSpec]:
        seen, out = set(), []
        for part in self._all_parts():
            for p in part.params():
                if p.name not in seen:
                    seen.add(p.name)
                    out.append(p)
        return out

    def kernel_groups(self) -> set[str]:
        return set().union(*(p.kernel_groups() for p in self._all_parts()))

    @property
    def graph_safe(self) -> bool:
        """May a step of this model be captured in a CUDA graph and replayed (see Part.graph_safe)?"""
        return all(p.graph_safe for p in self._all_parts())

    def parts_not_graph_safe(self) -> list[str]:
        out = []
        for p in self._all_parts():
            inner = getattr(p, "_parts", None)
            for q in (inner() if inner is not None else [p]):
                if not q.graph_safe:
                    out.append(type(q).__name__)
        return sorted(set(out))

    def notes(self, rt) -> list[str]:
        """Every part's notes, each once."""
        out: list[str] = []
        for part in self._all_parts():
            for n in part.notes(rt):
                if n not in out:
                    out.append(n)
        return out

    def bind(self, tensors: dict[str, torch.Tensor], rt, n_positions: int) -> None:
        for part in self._all_parts():
            part.bind(tensors, rt)
        for pe in self.position_encodings.values():
            pe.prepare(rt, n_positions)

    def register_cache(self, cache) -> None:
        """Tell the cache what every schedule entry keeps."""
        writes = []
        for e in self.spec.schedule:
            mixer = self.layers[e.layer].mixer
            cache.add_entry(mixer.cache_request(), mixer.state_bytes(), e.reads_cache_of)
            writes.append(e.reads_cache_of is None)
        cache.entry_writes = writes

    def forward(self, rt, step) -> torch.Tensor | None:
        """Runs the step's tokens; returns 32-bit logits [wanted rows, vocab] (None if none wanted)."""
        x = self.embedding.forward(rt, step)
        for pe in self.position_encodings.values():
            pe.on_embedding(rt, step, x)
        pending = None
        for idx, e in enumerate(self.spec.schedule):
            x, pending = self.layers[e.layer].forward(rt, step, x, pending, idx)
        if step.n_logit_rows == 0:
            return None
        h = self.final_norm.forward(rt, x, pending, rows=step.logit_rows)
        return self.head.forward(rt, step, h)

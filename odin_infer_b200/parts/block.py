"""How a layer's parts are arranged."""
from __future__ import annotations

from .base import Block, PartSpec, ResidualAdded, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x -> x + Mixer(Norm(x)) -> x + FeedForward(Norm(x)) (infer/forward.odin:51, :117-139).

    Each residual add is carried out by the norm that follows it: the block hands
    the update it has not yet added to whoever runs next."""

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec, norm_mixer: PartSpec, norm_feed_forward: PartSpec):
        self._mixer = build_part("mixer", mixer)
        self.ffn = build_part("feed_forward", feed_forward)
        self.norm_mixer = build_part("norm", norm_mixer)
        self.norm_ffn = build_part("norm", norm_feed_forward)

    @property
    def mixer(self):
        return self._mixer

    def _parts(self):
        return (self.norm_mixer, self._mixer, self.norm_ffn, self.ffn)

    def params(self):
        return [p for part in self._parts() for p in part.params()]

    def bind(self, tensors, rt):
        for part in self._parts():
            part.bind(tensors, rt)

    def kernel_groups(self):
        return set().union(*(p.kernel_groups() for p in self._parts()))

    def notes(self, rt):
        return [n for p in self._parts() for n in p.notes(rt)]

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self._parts())

    def forward(self, rt, step, x, pending, entry):
        mixer, ffn = self._mixer, self.ffn
        h = self.norm_mixer.forward(rt, x, pending)
        delta = mixer.forward(rt, step, h, entry, residual=x) if mixer.takes_residual else mixer.forward(rt, step, h, entry)
        h = self.norm_ffn.forward(rt, x, None if isinstance(delta, ResidualAdded) else delta)
        delta = ffn.forward(rt, step, h, residual=x) if ffn.takes_residual else ffn.forward(rt, step, h)
        return x, (None if isinstance(delta, ResidualAdded) else delta)

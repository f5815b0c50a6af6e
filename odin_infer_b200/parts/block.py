"""How a layer's parts are arranged."""
from __future__ import annotations

from .base import Block, NormedRows, PartSpec, build_part, register_part


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

    takes_next_norm = True

    @property
    def kernels_only(self):
        return all(p.kernels_only for p in self._parts())

    @property
    def first_norm(self):
        return self.norm_mixer

    def forward(self, rt, step, x, pending, entry, next_norm=None):
        """A part that takes sinks may carry out the add and the weighting of the norm after it
        inside its last product (few tokens); what it returns then is that norm's output."""
        mixer, ffn = self._mixer, self.ffn
        # rows that came through a sink may stay unscaled for a part that takes them so
        late = {"unscaled_ok": True} if isinstance(pending, NormedRows) and mixer.takes_sinks else {}
        h = self.norm_mixer.forward(rt, x, pending, **late)
        if mixer.takes_sinks:
            delta = mixer.forward(rt, step, h, entry, sink=self.norm_ffn.sink(x))
        else:
            delta = mixer.forward(rt, step, h, entry)
        late = {"unscaled_ok": True} if isinstance(delta, NormedRows) and ffn.takes_sinks else {}
        h = self.norm_ffn.forward(rt, x, delta, **late)
        if ffn.takes_sinks:
            delta = ffn.forward(rt, step, h, sink=next_norm.sink(x) if next_norm is not None else None)
        else:
            delta = ffn.forward(rt, step, h)
        return x, delta

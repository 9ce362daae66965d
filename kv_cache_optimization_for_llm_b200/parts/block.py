"""Arrangements of a mixer and a feed-forward inside one layer."""

from __future__ import annotations

from .base import Part
from .registry import register


@register("block", "prenorm")
class PreNormBlock(Part):
    """``h += mixer(norm1(h)); h += ff(norm2(h))`` (upstream: base/src/engine.cu:639-859).

    The float32 residual travels with the branch output that has not been added
    yet: each norm adds the pending ``delta`` first, so add and norm are one kernel,
    and the block hands its feed-forward output on as the next pending delta."""

    def __init__(self, mixer, mixer_norm, feed_forward, ff_norm):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.ff_norm = feed_forward, ff_norm

    def forward(self, residual, delta, batch, cache):
        x = self.mixer_norm.forward(residual, delta)
        a = self.mixer.forward(x, batch, cache)
        x = self.ff_norm.forward(residual, a)
        f = self.feed_forward.forward(x, batch)
        return residual, f

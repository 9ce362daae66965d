"""Arrangements of a mixer and a feed-forward inside one layer."""

from __future__ import annotations

import torch

from .base import Part
from .registry import register


@register("block", "prenorm")
class PreNormBlock(Part):
    """``h += mixer(norm1(h)); h += ff(norm2(h))`` (upstream: base/src/engine.cu:639-859).

    The float32 residual travels with the branch output that has not been added
    yet: each norm adds the pending ``delta`` first, so add and norm are one kernel,
    and the block hands its feed-forward output on as the next pending delta.

    A mixer or feed-forward with ``fuses_residual = True`` goes one step further (bfloat16
    only; the 32-bit path keeps every formula as it stands).  When the block is built, the
    part multiplies the weight of the norm in front of it into its own input matrices
    (``fold_input_scale``) and the norm becomes weightless.  ``forward`` then may get ``x`` as
    an ``ops.PendingNorm``, carried out by the part's first product, and gets the residual as
    ``into=``, which its last product may add to itself, returning an ``ops.Folded``."""

    # the parts this arrangement takes, by name, and the family each is looked up in
    part_families = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "ff_norm": "norm"}

    def __init__(self, parts):
        self.parts = dict(parts)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.ff_norm = parts["feed_forward"], parts["ff_norm"]
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.ff_norm)):
            if (getattr(part, "fuses_residual", False) and part.ctx.dtype == torch.bfloat16
                    and hasattr(norm, "give_up_weight") and norm.weight is not None):
                part.fold_input_scale(norm.give_up_weight())

    def cache_spec(self):
        """What this layer asks of the cache: its mixer's wish."""
        return self.mixer.cache_spec()

    def forward(self, residual, delta, batch, cache):
        if getattr(self.mixer, "fuses_residual", False):
            x = self.mixer_norm.forward(residual, delta, lazy=True)
            a = self.mixer.forward(x, batch, cache, into=residual)
        else:
            a = self.mixer.forward(self.mixer_norm.forward(residual, delta), batch, cache)
        if getattr(self.feed_forward, "fuses_residual", False):
            x = self.ff_norm.forward(residual, a, lazy=True)
            f = self.feed_forward.forward(x, batch, into=residual)
        else:
            f = self.feed_forward.forward(self.ff_norm.forward(residual, a), batch)
        return residual, f

"""Position encodings."""

from __future__ import annotations

import math

import torch

from .base import Part
from .registry import register


def rope_inv_freq(head_dim: int, theta: float, scaling) -> torch.Tensor:
    """Rotary frequencies in float64: ``1/theta^(2i/d)``, then the llama3 rescale by
    wavelength band: long waves divided by ``factor``, short ones kept, a linear
    blend between (upstream computes the same in float32, base/src/kernels.cu:58-83)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / head_dim)
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type", "llama3"))
    if kind != "llama3":
        raise ValueError(f"rope scaling of type {kind!r} is not known to this position encoding "
                         "(known: none, 'llama3')")
    factor = float(scaling["factor"])
    low_ff, high_ff = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (orig / wavelen - low_ff) / (high_ff - low_ff)
    blended = (1.0 - smooth) * (inv / factor) + smooth * inv
    out = torch.where(wavelen > orig / low_ff, inv / factor,
                      torch.where(wavelen >= orig / high_ff, blended, inv))
    return out


@register("position", "rope")
class RotaryEncoding(Part):
    """Rotate-half rotary encoding with optional llama3 frequency scaling.

    Holds float32 tables ``cos, sin [max_positions, rotary_dim/2]`` whose angles
    ``pos * inv_freq`` are formed in float64 (upstream: float32 tables with each
    value stored twice, base/src/kernels.cu:85-105).  The rotation itself runs in
    the kernel that also writes keys and values to the cache.
    params: head_dim, rotary_dim, theta, scaling (dict or None)."""

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim > params["head_dim"]:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim")
        key = ("rope", self.rotary_dim, float(params["theta"]),
               tuple(sorted((k, str(v)) for k, v in (params["scaling"] or {}).items())), ctx.max_positions)
        if key not in ctx.shared:
            inv = rope_inv_freq(self.rotary_dim, params["theta"], params["scaling"])
            ang = torch.arange(ctx.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            ctx.shared[key] = (ang.cos().to(torch.float32).to(ctx.device).contiguous(),
                               ang.sin().to(torch.float32).to(ctx.device).contiguous())
        self.cos, self.sin = ctx.shared[key]

    def tables(self):
        return self.cos, self.sin

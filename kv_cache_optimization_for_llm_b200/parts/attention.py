"""Attention mixers."""

from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.specs import PagedKVSpec
from ..weights.loader import WeightSpec
from .base import Part
from .registry import lookup, register


@register("mixer", "attention")
class GroupedQueryAttention(Part):
    """Causal grouped-query attention over the paged cache.

    q, k, v come from one product with the row-stacked [q; k; v] matrix; q and k are
    rotated, k and v go to the request's pages, and every token attends to the keys
    of its own request up to its position (the newest ``window`` of them when a
    window is set), read from the pages.  Then the output projection.
    Upstream: base/src/engine.cu:653-762; it attends over the step's own packed
    keys in prefill and over the cache in decode, in separate passes.
    params: hidden_size, num_heads, num_kv_heads, head_dim, window (None or int),
    position (a PartSpec of the position family, or None)."""

    @classmethod
    def weight_specs(cls, params):
        h, nq, nkv, d = (params[k] for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim"))
        return {"q": WeightSpec((nq * d, h)), "k": WeightSpec((nkv * d, h)),
                "v": WeightSpec((nkv * d, h)), "o": WeightSpec((h, nq * d))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        mods = ["elementwise", "attention"]
        if dtype == torch.bfloat16 and params["head_dim"] in (64, 128):
            mods += ["flash_attention", "decode_attention"]
        mods += ["gemm_f32"] if dtype == torch.float32 else ["gemm_bf16", "gemm_bf16_wide"]
        return tuple(mods)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.nq, self.nkv, self.d = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot be grouped over {self.nkv} key/value heads")
        if self.d % 16 or self.d > 256:
            raise ValueError(f"head_dim {self.d} is refused: the attention kernels take multiples of 16 up to 256")
        self.window = params.get("window") or None
        self.scale = 1.0 / math.sqrt(self.d)
        self.qkv = torch.cat([weights["q"], weights["k"], weights["v"]], dim=0).contiguous()
        self.o = weights["o"]
        pos = params.get("position")
        self.position = None
        if pos is not None:
            self.position = (ctx.make("position", pos) if ctx.make is not None
                             else lookup("position", pos.kind)(pos.params, {}, ctx))

    fuses_residual = True

    def fold_input_scale(self, scale):
        """Multiplies ``scale`` [hidden] (the weight of the norm in front) into the input
        columns of the q, k, v matrix, so that the norm itself can go without."""
        self.qkv = (self.qkv.float() * scale.float()[None, :]).to(self.qkv.dtype).contiguous()

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window)

    def activation_widths(self):
        """Elements per token of the tensors one call produces: q|k|v, the attention output, and
        the projected output (or its bfloat16 copy with the partial sums of squares)."""
        hidden = self.o.shape[0]
        return [(self.nq + 2 * self.nkv) * self.d, self.nq * self.d, 2 * hidden]

    def query_tile_heights(self):
        """Tokens per tile of the tensor-core attention for prompt portions (bfloat16, head sizes
        it takes): the step's batch lays the tiles out for them."""
        if self.ctx.dtype != torch.bfloat16 or self.d not in (64, 128):
            return []
        g = self.nq // self.nkv
        return [ops.flash_tokens_per_tile(g, False), ops.flash_tokens_per_tile(g, True)]

    def forward(self, x, batch, cache, into=None):
        qkv = ops.linear(x, self.qkv)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rot = self.position.rotary_dim if self.position is not None else 0
        table = batch.block_tables[cache.group]
        a = ops.attention_step(qkv, cache.k, cache.v, cache.write, table, batch, self.nq, self.nkv, self.d,
                               self.scale, self.window, self.ctx.max_positions, cos, sin, rot)
        return ops.linear(a, self.o, into=into)

"""Feed-forward parts."""

from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("feed_forward", "swiglu")
class SwiGLU(Part):
    """``down( silu(gate(x)) * up(x) )``, no bias (upstream: base/src/engine.cu:780-855,
    base/src/kernels.cu:45-52).  gate and up are stored as one [2*I, H] matrix so
    one product feeds the activation kernel.  params: hidden_size, intermediate_size."""

    @classmethod
    def weight_specs(cls, params):
        h, i = params["hidden_size"], params["intermediate_size"]
        return {"gate": WeightSpec((i, h)), "up": WeightSpec((i, h)), "down": WeightSpec((h, i))}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise", "gemm_f32" if dtype == torch.float32 else "gemm_bf16")

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.gate_up = torch.cat([weights["gate"], weights["up"]], dim=0).contiguous()
        self.down = weights["down"]

    def forward(self, x, batch):
        gu = ops.linear(x, self.gate_up)
        a = ops.silu_mul(gu)
        return ops.linear(a, self.down)

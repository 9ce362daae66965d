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
        return ("elementwise",) + (("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide"))

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        inter = int(params["intermediate_size"])
        # gate and up rows alternate in blocks, so that a 128-row tile of the product holds
        # 64 gate features and the 64 up features of the same indices and the activation
        # can be the product's epilogue; widths that are no multiple of 64 keep [gate | up]
        self.block = 64 if inter % 64 == 0 else inter
        g, u = weights["gate"], weights["up"]
        if self.block == inter:
            self.gate_up = torch.cat([g, u], dim=0).contiguous()
        else:
            nb, h = inter // self.block, g.shape[1]
            self.gate_up = torch.stack([g.view(nb, self.block, h), u.view(nb, self.block, h)], dim=1) \
                .reshape(2 * inter, h).contiguous()
        self.down = weights["down"]

    fuses_residual = True

    def fold_input_scale(self, scale):
        """Multiplies ``scale`` [hidden] (the weight of the norm in front) into the input
        columns of the gate and up matrix, so that the norm itself can go without."""
        self.gate_up = (self.gate_up.float() * scale.float()[None, :]).to(self.gate_up.dtype).contiguous()

    def activation_widths(self):
        """Elements per token of the tensors one call produces: gate|up (when the activation is a
        kernel of its own), the activation, and the output (or its bfloat16 copy with sums)."""
        inter, hidden = self.gate_up.shape[0] // 2, self.down.shape[0]
        return [2 * inter, inter, 2 * hidden]

    def forward(self, x, batch, into=None):
        a = ops.linear_swiglu(x, self.gate_up, self.block)
        return ops.linear(a, self.down, into=into)

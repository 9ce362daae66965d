"""RMSNorm with the residual add fused in front of it."""

from __future__ import annotations

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Part):
    """``y = v / sqrt(mean(v^2) + eps) * w`` over the whole width, plain weight
    (upstream: base/src/kernels.cu:10-36), where ``v = residual + delta`` is summed
    and kept in float32 (upstream adds in a second kernel and keeps bfloat16,
    base/src/kernels.cu:38-43).  params: size, eps."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": WeightSpec((params["size"],), "vector")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.eps = float(params["eps"])
        self.weight = weights["weight"]

    def forward(self, residual, delta=None, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.ctx.dtype, rows)

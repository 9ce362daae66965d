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
        self.size = int(params["size"])
        self.weight = weights["weight"]

    def activation_widths(self):
        return [self.size]

    def give_up_weight(self):
        """Hands the weight to a part that multiplies it into its own matrices
        (``fold_input_scale``); the norm is weightless from then on."""
        w, self.weight = self.weight, None
        return w

    def forward(self, residual, delta=None, rows=None, lazy=False):
        if isinstance(delta, ops.Folded):
            # the branch before this norm has added its output itself and left the sums of squares
            if lazy and rows is None and self.weight is None:
                return ops.PendingNorm(residual, delta.xb, delta.sumsq, self.eps, self.ctx.dtype)
            delta = None
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.ctx.dtype, rows)

"""Token embedding and the LM head."""

from __future__ import annotations

from .. import ops
from ..weights.loader import WeightSpec
from .base import Part
from .registry import register


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``residual[t] = table[token[t]]``, no scaling (upstream: base/src/kernels.cu:279-287).
    The residual stream starts, and stays, in float32.  params: vocab_size, hidden_size."""

    @classmethod
    def weight_specs(cls, params):
        return {"table": WeightSpec((params["vocab_size"], params["hidden_size"]), "matrix")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        return ("elementwise",)

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.table = weights["table"]

    def forward(self, batch):
        return ops.embed_gather(self.table, batch.token_ids, batch.status, batch.sampled)


@register("head", "linear_head")
class LinearHead(Part):
    """``logits = x . W^T`` in float32 output, W either its own tensor or the embedding
    table when tied (upstream: base/src/engine.cu:872-890, always tied, bfloat16
    logits).  params: vocab_size, hidden_size."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": WeightSpec((params["vocab_size"], params["hidden_size"]), "matrix")}

    @classmethod
    def kernel_modules(cls, params, dtype):
        import torch
        return ("gemm_f32",) if dtype == torch.float32 else ("gemm_bf16", "gemm_bf16_wide")

    def __init__(self, params, weights, ctx):
        super().__init__(params, weights, ctx)
        self.weight = weights["weight"]

    def forward(self, x):
        import torch
        return ops.linear(x, self.weight, out_dtype=torch.float32)

"""A model put together from parts according to its description."""

from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from ..models.spec import ModelSpec, PartSpec, block_part_families, expected_weights
from ..parts import BuildContext, lookup
from ..weights.loader import to_compute


class DecoderModel:
    """Embedding, the scheduled layers, final norm and head.

    ``forward`` runs exactly the tokens of the batch, reads and writes the cache
    through each schedule entry's binding, and returns float32 logits at
    ``batch.logit_rows`` only."""

    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], ctx: BuildContext):
        spec.validate()
        self.spec, self.ctx = spec, ctx
        wanted = expected_weights(spec)
        # One device copy per checkpoint tensor, however many parts name it.
        dev: Dict[str, torch.Tensor] = {}
        for name, ws in wanted.items():
            dev[name] = to_compute(tensors[name], ws, ctx.dtype, ctx.device)

        def make(family: str, ps: PartSpec):
            cls = lookup(family, ps.kind)
            return cls(ps.params, {role: dev[name] for role, name in ps.weights.items()}, ctx)

        ctx.make = make     # parts that hold further parts build them through this
        self.embedding = make("embedding", spec.embedding)
        self.layers = []
        for ls in spec.layers:
            block_cls = lookup("block", ls.block)
            self.layers.append(block_cls({name: make(family, ls.parts[name])
                                          for name, family in block_part_families(ls.block).items()}))
        self.final_norm = make("norm", spec.final_norm)
        self.head = make("head", spec.lm_head)
        self.schedule = list(spec.schedule)

    def cache_specs(self):
        """Per schedule entry: what its mixer asks of the cache, and whose cache it reads."""
        specs = [self.layers[e.layer].cache_spec() for e in self.schedule]
        return specs, [e.cache_of for e in self.schedule]

    def kernel_modules(self) -> List[str]:
        return kernel_modules_of(self.spec, self.ctx.dtype)

    def forward(self, batch, cache, arena=None) -> torch.Tensor:
        """``arena``: the step's memory (engine/arena.py).  With it, every tensor that the parts
        produce through ``ops`` lies in it: the residual and the logits for the length of the
        step, a layer's tensors until the layer after the next begins."""
        from .. import ops
        if arena is None:
            with ops.use_current_stream():
                return self._forward(batch, cache, None)
        with ops.use_current_stream(), ops.use_arena(arena):
            return self._forward(batch, cache, arena)

    def _forward(self, batch, cache, arena) -> torch.Tensor:
        if arena is not None:
            arena.begin_step()
        residual = self.embedding.forward(batch)
        delta = None
        for i, entry in enumerate(self.schedule):
            if arena is not None:
                arena.begin_layer()
            residual, delta = self.layers[entry.layer].forward(residual, delta, batch, cache.binding(i))
        if arena is not None:
            arena.end_layers()
        if batch.num_logits == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        x = self.final_norm.forward(residual, delta, rows=batch.logit_rows)
        return self.head.forward(x)

    def arena_bytes(self, max_tokens: int, max_logit_rows: int):
        """(bytes that live for a whole step, bytes that one layer produces) for steps of up to
        ``max_tokens`` tokens with up to ``max_logit_rows`` rows of logits: the residual in
        float32, the picked rows and their logits; and per layer the widths its parts declare
        (``activation_widths``; a part that declares none is taken as eight rows of the model's
        width) in the compute precision, plus a fifth."""
        h, v = self.spec.hidden_size, self.spec.vocab_size
        step = 4 * max_tokens * h + max_logit_rows * 4 * (h + v) + (1 << 16)
        per_layer = 0
        for block in self.layers:
            widths = 0
            for part in getattr(block, "parts", {}).values():
                declared = getattr(part, "activation_widths", None)
                widths += sum(declared()) if declared is not None else 8 * h
            per_layer = max(per_layer, widths or 32 * h)
        esize = 4 if self.ctx.dtype == torch.float32 else 2
        layer = int(1.2 * esize * max_tokens * per_layer) + (1 << 16)
        return step, layer

    def query_tile_heights(self):
        """Tokens per query tile that the model's mixers cut a step's runs of tokens into."""
        out = set()
        for block in self.layers:
            for part in getattr(block, "parts", {}).values():
                fn = getattr(part, "query_tile_heights", None)
                if fn is not None:
                    out.update(fn())
        return sorted(out)


def kernel_modules_of(spec: ModelSpec, dtype: torch.dtype) -> List[str]:
    """The kernel modules (csrc/kernels/<name>.cu) that the model's parts launch."""
    from ..models.spec import iter_parts
    mods: List[str] = []
    for family, ps in iter_parts(spec):
        if family == "block":
            continue
        cls = lookup(family, ps.kind)
        for m in (cls.kernel_modules(ps.params, dtype) if hasattr(cls, "kernel_modules") else ()):
            if m not in mods:
                mods.append(m)
    return mods

"""What every part has in common.

A part is built from its ``params`` (sizes and constants), the tensors named by its
roles, and a :class:`BuildContext` (compute dtype, device, limits).  It knows
nothing of the model it sits in.  Interfaces by family:

* norm:          ``forward(residual, delta, rows=None) -> normed``; adds ``delta`` into the
                 float32 ``residual`` first (in place) when it is given
* mixer:         ``cache_spec() -> PagedKVSpec | SlotStateSpec | None`` and
                 ``forward(x, batch, cache) -> delta``
* feed_forward:  ``forward(x, batch) -> delta``
* position:      whatever its mixer uses (rope: ``tables() -> (cos, sin)``)
* block:         ``part_families`` (name -> family of the parts it arranges), built from a
                 mapping name -> part; ``cache_spec()`` (what the layer asks of the cache) and
                 ``forward(residual, delta, batch, cache) -> (residual, delta)``
* a part that holds further parts (a ``PartSpec`` among its params) builds them with
  ``ctx.make(family, spec)``, which also hands them their tensors
* a mixer or feed-forward may set ``fuses_residual = True``; it then has
  ``fold_input_scale(vector)``, and its ``forward`` also takes ``into=residual`` and may get
  ``x`` as an ``ops.PendingNorm`` (see the prenorm block)
* embedding:     ``forward(batch) -> residual``  (float32 [T, hidden])
* head:          ``forward(x) -> logits``  (float32 [rows, vocab])
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional

import torch

from ..weights.loader import WeightSpec


@dataclass
class BuildContext:
    dtype: torch.dtype          # activations, weights and cache: bfloat16 or float32
    device: torch.device
    max_positions: int          # positions the engine may ever see
    status: torch.Tensor        # [1] int32 device word for kernel-side error reports
    shared: dict = field(default_factory=dict)  # tables shared between equal parts
    make: Optional[Callable] = None  # (family, PartSpec) -> the built part with its tensors; set by the model


class Part:
    family = "?"
    kind = "?"

    @classmethod
    def weight_specs(cls, params: Mapping) -> Dict[str, WeightSpec]:
        """role -> shape/kind of every tensor the part needs."""
        return {}

    @classmethod
    def kernel_modules(cls, params: Mapping, dtype: torch.dtype):
        """Names of the kernel modules (csrc/kernels/<name>.cu) the part launches."""
        return ()

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], ctx: BuildContext):
        self.params = dict(params)
        self.ctx = ctx

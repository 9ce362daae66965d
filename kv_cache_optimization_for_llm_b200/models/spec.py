"""The description of a model as data: which parts each layer is made of, with
which sizes, which checkpoint tensors feed them, and in which order layers run.

An architecture (``models/llama.py``) turns its typed configuration into a
:class:`ModelSpec`; everything below that (parts, cache, step function) reads only
the spec and knows no architecture.  Upstream has no such layer: its single model
is a sequence of launches written out by hand (base/src/engine.cu:639-890).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..weights.loader import WeightSpec


@dataclass
class PartSpec:
    """One part: ``kind`` picks the class from its family's registry, ``params`` holds
    its sizes and constants, ``weights`` maps the part's tensor roles to checkpoint
    tensor names."""
    kind: str
    params: dict = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """A layer: a block arrangement around a mixer and a feed-forward with their norms."""
    block: str
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    ff_norm: PartSpec


@dataclass
class ScheduleEntry:
    """One application of a layer.  ``cache_of``: index of an earlier schedule entry
    whose cache this application reads instead of keeping one of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    lm_head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None and not 0 <= e.cache_of < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                 "which must be an earlier entry")
            if e.cache_of is not None and self.schedule[e.cache_of].cache_of is not None:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, "
                                 "which keeps none of its own")


def iter_parts(spec: ModelSpec):
    """(family, PartSpec) of every part of the model, nested ones (a mixer's position
    encoding) included."""
    yield "embedding", spec.embedding
    for layer in spec.layers:
        yield "block", PartSpec(layer.block)
        yield "mixer", layer.mixer
        pos = layer.mixer.params.get("position")
        if isinstance(pos, PartSpec):
            yield "position", pos
        yield "norm", layer.mixer_norm
        yield "feed_forward", layer.feed_forward
        yield "norm", layer.ff_norm
    yield "norm", spec.final_norm
    yield "head", spec.lm_head


def expected_weights(spec: ModelSpec) -> Dict[str, WeightSpec]:
    """Checkpoint tensor name -> shape and kind, over every part.  A tensor that two
    parts name (a tied head) must be wanted with one shape."""
    from ..parts import registry as parts
    out: Dict[str, WeightSpec] = {}
    for family, ps in iter_parts(spec):
        if family in ("block", "position"):
            continue
        cls = parts.lookup(family, ps.kind)
        for role, ws in cls.weight_specs(ps.params).items():
            if role not in ps.weights:
                raise ValueError(f"part {family}/{ps.kind} needs a tensor for role {role!r}, "
                                 f"the spec names only {sorted(ps.weights)}")
            name = ps.weights[role]
            if name in out and out[name].shape != ws.shape:
                raise ValueError(f"tensor {name} is wanted with shapes {out[name].shape} and {ws.shape}")
            out.setdefault(name, ws)
    return out

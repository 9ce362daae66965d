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
    tensor names.  A part may hold further parts among its ``params`` (a mixer its
    position encoding, a mixer a norm of its own, a feed-forward its experts): such a
    nested part belongs to the family that its ``family`` names, or, if that is empty,
    to the family called like the key it sits under."""
    kind: str
    params: dict = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)
    family: str = ""


@dataclass
class LayerSpec:
    """A layer: a block arrangement and the parts it arranges, by the names the block
    gives them.  Which names a block takes, and of which family each is, is the block
    class's ``part_families`` (the pre-norm block: mixer, mixer_norm, feed_forward,
    ff_norm); a block with further norms or a third branch simply names more."""
    block: str
    parts: Dict[str, PartSpec] = field(default_factory=dict)


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


def _with_nested(family: str, ps: PartSpec):
    """The part, then every part nested in its params (directly, or in lists, tuples and
    dicts there), depth first."""
    yield family, ps

    def walk(key, value):
        if isinstance(value, PartSpec):
            yield from _with_nested(value.family or key, value)
        elif isinstance(value, (list, tuple)):
            for v in value:
                yield from walk(key, v)
        elif isinstance(value, dict):
            for k, v in value.items():
                yield from walk(k, v)

    for key, value in ps.params.items():
        yield from walk(key, value)


def block_part_families(block_kind: str) -> Dict[str, str]:
    """name -> family of the parts that a block arrangement takes."""
    from ..parts import registry as parts
    cls = parts.lookup("block", block_kind)
    fam = getattr(cls, "part_families", None)
    if not fam:
        raise ValueError(f"block {block_kind!r} does not say which parts it takes (part_families)")
    return dict(fam)


def iter_parts(spec: ModelSpec):
    """(family, PartSpec) of every part of the model, nested ones included, whatever
    their family and however deep."""
    yield from _with_nested("embedding", spec.embedding)
    for i, layer in enumerate(spec.layers):
        yield "block", PartSpec(layer.block)
        families = block_part_families(layer.block)
        missing = sorted(set(families) - set(layer.parts))
        extra = sorted(set(layer.parts) - set(families))
        if missing or extra:
            raise ValueError(f"layer {i}: block {layer.block!r} takes the parts {sorted(families)}; "
                             f"missing {missing}, not taken {extra}")
        for name, family in families.items():
            yield from _with_nested(family, layer.parts[name])
    yield from _with_nested("norm", spec.final_norm)
    yield from _with_nested("head", spec.lm_head)


def expected_weights(spec: ModelSpec) -> Dict[str, WeightSpec]:
    """Checkpoint tensor name -> shape and kind, over every part.  A tensor that two
    parts name (a tied head) must be wanted with one shape."""
    from ..parts import registry as parts
    out: Dict[str, WeightSpec] = {}
    for family, ps in iter_parts(spec):
        if family == "block":
            continue
        cls = parts.lookup(family, ps.kind)
        wanted = cls.weight_specs(ps.params) if hasattr(cls, "weight_specs") else {}
        for role, ws in wanted.items():
            if role not in ps.weights:
                raise ValueError(f"part {family}/{ps.kind} needs a tensor for role {role!r}, "
                                 f"the spec names only {sorted(ps.weights)}")
            name = ps.weights[role]
            if name in out and out[name].shape != ws.shape:
                raise ValueError(f"tensor {name} is wanted with shapes {out[name].shape} and {ws.shape}")
            out.setdefault(name, ws)
    return out

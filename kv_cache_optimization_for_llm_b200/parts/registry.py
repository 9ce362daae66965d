"""Registries of parts, one per family.  A model description names a part by
(family, kind); a new kind is one ``@register`` away and needs no change here."""

from __future__ import annotations

from typing import Dict

FAMILIES = ("embedding", "mixer", "feed_forward", "norm", "position", "block", "head")
_REG: Dict[str, Dict[str, type]] = {f: {} for f in FAMILIES}


def register(family: str, kind: str):
    if family not in _REG:
        raise ValueError(f"unknown part family {family!r}; families: {FAMILIES}")

    def deco(cls):
        _REG[family][kind] = cls
        cls.family, cls.kind = family, kind
        return cls
    return deco


def lookup(family: str, kind: str) -> type:
    _load_builtin()
    try:
        return _REG[family][kind]
    except KeyError:
        raise ValueError(f"no {family} part of kind {kind!r} is registered; known: "
                         + ", ".join(sorted(_REG.get(family, {})))) from None


def known(family: str):
    _load_builtin()
    return sorted(_REG[family])


def _load_builtin() -> None:
    from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401

"""One registry from an architecture's name (``architectures[0]`` of config.json) to
its typed configuration and its model description.  Upstream has one hard-wired
model and no registry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .models.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed configuration
    build_spec: Callable[[Any], ModelSpec]             # typed configuration -> model description


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config, build_spec) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def known_architectures():
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin() -> None:
    from .models import llama  # noqa: F401  (registers itself)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    _load_builtin()
    archs = config_dict.get("architectures") or []
    if not archs:
        raise ValueError("config.json: 'architectures' is missing or empty; known: "
                         + ", ".join(sorted(_ARCHITECTURES)))
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is not registered; known: " + ", ".join(sorted(_ARCHITECTURES)))
    return _ARCHITECTURES[name]

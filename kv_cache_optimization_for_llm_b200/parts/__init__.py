from .base import BuildContext, Part
from .registry import known, lookup, register

__all__ = ["BuildContext", "Part", "known", "lookup", "register"]

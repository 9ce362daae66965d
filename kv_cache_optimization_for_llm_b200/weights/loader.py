"""Loads a model's tensors by name and checks them against what the model expects.

Upstream fills its pointers by name without any check: a missing tensor ends in an
uncaught exception and a wrong shape goes unnoticed (base/src/model.cu:66-82).
Here one error lists everything at once: missing tensors, unexpected ones and
wrong shapes.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsError, read_header, read_tensors


@dataclass(frozen=True)
class WeightSpec:
    """What a part expects of one tensor.  ``kind``: 'matrix' (cast to the compute
    dtype), 'vector' (kept in 32-bit: norm weights) or 'table' (integers, int32)."""
    shape: Tuple[int, ...]
    kind: str = "matrix"


class WeightError(ValueError):
    """The checkpoint does not hold what the model needs."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = [f"the weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " +
                         ", ".join(f"{n}: stored {tuple(g)}, wanted {tuple(w)}" for n, g, w in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " +
                         ", ".join(f"{n}: stored {d}, wanted {w}" for n, d, w in self.wrong_dtype))
        super().__init__("\n".join(lines))


def _files(model_dir: Path):
    index = model_dir / "model.safetensors.index.json"
    single = model_dir / "model.safetensors"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        return sorted({model_dir / f for f in weight_map.values()})
    if single.exists():
        return [single]
    raise FileNotFoundError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")


def check_and_load(model_dir, expected: Mapping[str, WeightSpec]) -> Dict[str, torch.Tensor]:
    """Returns name -> CPU tensor in the stored dtype for exactly the expected names."""
    model_dir = Path(model_dir)
    files = _files(model_dir)
    stored = {}
    for f in files:
        header, _ = read_header(f)
        for name, meta in header.items():
            stored[name] = (f, meta)
    missing = [n for n in expected if n not in stored]
    unexpected = [n for n in stored if n not in expected]
    wrong_shape, wrong_dtype = [], []
    for n, spec in expected.items():
        if n not in stored:
            continue
        meta = stored[n][1]
        if tuple(meta["shape"]) != tuple(spec.shape):
            wrong_shape.append((n, tuple(meta["shape"]), tuple(spec.shape)))
        is_int = meta["dtype"] in ("I32", "I64", "I16", "I8", "U8", "BOOL")
        if (spec.kind == "table") != is_int:
            wrong_dtype.append((n, meta["dtype"], "integer" if spec.kind == "table" else "floating point"))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(str(model_dir), missing, unexpected, wrong_shape, wrong_dtype)
    out: Dict[str, torch.Tensor] = {}
    for f in files:
        out.update(read_tensors(f, names=set(expected)))
    return out


def to_compute(t: torch.Tensor, spec: WeightSpec, dtype: torch.dtype, device) -> torch.Tensor:
    """Storage -> what the kernels read.  Matrices take the compute dtype (a
    bfloat16 matrix stays bfloat16 in the serving path, becomes float32 exactly in
    the 32-bit path); vectors are kept in 32-bit; integer tables become int32."""
    if spec.kind == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    if spec.kind == "vector":
        return t.to(device=device, dtype=torch.float32).contiguous()
    return t.to(device=device, dtype=dtype).contiguous()

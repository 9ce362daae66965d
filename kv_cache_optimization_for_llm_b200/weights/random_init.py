"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed.  Upstream has no such mode; it always loads the
real checkpoint (base/src/model.cu:15-84).

Matrices are N(0, std), norm weights 1 + N(0, std), drawn in float32 from one
generator in the order of the tensor names, so a (configuration, seed, std) names
one model exactly.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch

from .loader import WeightSpec
from .safetensors_io import write_tensors


def random_tensors(expected: Mapping[str, WeightSpec], seed: int, std: float = 0.02,
                   storage_dtype: torch.dtype = torch.float32):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.kind == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
        if spec.kind == "vector":
            t = t + 1.0
        out[name] = t.to(storage_dtype)
    return out


def random_tensors_on_device(expected: Mapping[str, WeightSpec], seed: int, std: float, dtype: torch.dtype, device):
    """The same distribution drawn on the device in the compute dtype, for runs that
    need a large random model and no file (benchmarks)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.kind == "table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * std
        out[name] = (t + 1.0) if spec.kind == "vector" else t.to(dtype)
    return out


def write_random_model(model_dir, config_dict: dict, seed: int, std: float = 0.02,
                       storage_dtype: str = "float32") -> Path:
    """Builds the model that ``config_dict`` names (through the registry, as a
    loaded model would be) and writes random tensors for every name it expects."""
    from ..registry import resolve_architecture
    arch = resolve_architecture(config_dict)
    spec = arch.build_spec(arch.parse_config(config_dict))
    from ..models.spec import expected_weights
    expected = expected_weights(spec)
    st = {"float32": torch.float32, "bfloat16": torch.bfloat16}[storage_dtype]
    tensors = random_tensors(expected, seed, std, st)
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    cfg = dict(config_dict)
    cfg["torch_dtype"] = storage_dtype
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    write_tensors(model_dir / "model.safetensors", tensors,
                  metadata={"format": "pt", "seed": seed, "std": std})
    return model_dir

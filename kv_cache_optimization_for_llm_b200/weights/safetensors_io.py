"""Reads and writes the safetensors container: a u64 header length, a JSON header
with dtype, shape and byte range per tensor, then the raw payload
(the format upstream reads in base/src/model.cu:33-64, where only the start
offsets are used and neither dtype nor shape is looked at).
"""

from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Mapping, Tuple

import numpy as np
import torch

_TORCH = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _TORCH.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path) -> Tuple[Dict[str, dict], int]:
    """Returns (tensor name -> {dtype, shape, data_offsets}, offset of the payload)."""
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file ({size} bytes)")
        try:
            header = json.loads(f.read(n))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
    header.pop("__metadata__", None)
    for name, meta in header.items():
        lo, hi = meta["data_offsets"]
        if meta["dtype"] not in _TORCH:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        want = int(np.prod(meta["shape"], dtype=np.int64)) * torch.empty((), dtype=_TORCH[meta["dtype"]]).element_size()
        if hi - lo != want:
            raise SafetensorsError(f"{path}: tensor {name!r} covers {hi - lo} bytes, its shape and dtype need {want}")
        if 8 + n + hi > size:
            raise SafetensorsError(f"{path}: tensor {name!r} ends at byte {8 + n + hi}, the file has {size} (truncated?)")
    return header, 8 + n


def read_tensors(path, names=None) -> Dict[str, torch.Tensor]:
    """Loads tensors (all, or the named ones) in their stored dtype, on the CPU."""
    header, base = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    for name, meta in header.items():
        if names is not None and name not in names:
            continue
        lo, hi = meta["data_offsets"]
        dt = _TORCH[meta["dtype"]]
        if hi == lo:
            out[name] = torch.empty(meta["shape"], dtype=dt)
            continue
        raw = np.fromfile(path, dtype=np.uint8, count=hi - lo, offset=base + lo)
        out[name] = torch.from_numpy(raw).view(dt).reshape(meta["shape"])
    return out


def write_tensors(path, tensors: Mapping[str, torch.Tensor], metadata=None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)

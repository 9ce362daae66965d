"""What a mixer asks of the cache, and what it is handed back at each step."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values that grow with the sequence, kept in pages.  ``window``: only
    the newest ``window`` keys are ever read, older pages may be given back."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotStateSpec:
    """State of fixed size per request, kept in the request's state slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PagedKVBinding:
    """A schedule entry's view of its pages: ``k`` and ``v`` are
    [num_pages, num_kv_heads, page_size, head_dim]; the block tables of the step's
    requests are ``batch.block_tables[group]``.  ``write`` is False for an entry that
    reads another entry's cache."""
    k: torch.Tensor
    v: torch.Tensor
    group: int
    page_size: int
    write: bool = True


@dataclass
class SlotStateBinding:
    """A schedule entry's per-request state: ``state[slot]`` with the step's slots in
    ``batch.slots``.  A request whose portion starts at position 0 has to be reset
    by the mixer (``batch.req_start``)."""
    state: torch.Tensor
    write: bool = True

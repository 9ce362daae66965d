"""The cache as the model sees it: device tensors for pages and state slots, laid out
from what the mixers ask for, with the native manager keeping the books.

Upstream keeps one pool of 32 KiB pages, each holding 16 tokens of one layer
(K[16][512] then V[16][512]), and a block table per slot and layer
(paged_attention/src/config.h:181-193, paged_attention/src/engine.cu:176-254).
Here a page id covers every layer of its group: the group's tensor is
[entries, 2, num_pages, kv_heads, page_size, head_dim], so a (page, head) tile is one
contiguous run and the block table is one row per request.  Mixers with equal
needs share a group; mixers with other needs (another head shape, a window) get a
group, a pool and tables of their own.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import build
from .specs import PagedKVBinding, PagedKVSpec, SlotStateBinding, SlotStateSpec


def host_runtime():
    return build.load_host()


class PagedCache:
    def __init__(self, entry_specs: Sequence[Optional[object]], cache_of: Sequence[Optional[int]],
                 page_size: int, num_pages: int, num_slots: int, max_model_len: int,
                 dtype: torch.dtype, device, allocate: bool = True):
        """``entry_specs[i]``: what schedule entry i's mixer asks for (PagedKVSpec,
        SlotStateSpec or None).  ``cache_of[i]``: entry whose cache entry i reads."""
        self.page_size, self.num_pages, self.num_slots = int(page_size), int(num_pages), int(num_slots)
        self.dtype, self.device = dtype, torch.device(device)
        host = host_runtime()
        group_keys: List[Tuple] = []
        self.entry_group: List[Optional[Tuple[int, int]]] = []  # (group, index inside it)
        counts: List[int] = []
        for i, spec in enumerate(entry_specs):
            if cache_of[i] is not None or not isinstance(spec, PagedKVSpec):
                self.entry_group.append(None)
                continue
            key = (spec.num_kv_heads, spec.head_dim, spec.window or 0)
            if key not in group_keys:
                group_keys.append(key)
                counts.append(0)
            g = group_keys.index(key)
            self.entry_group.append((g, counts[g]))
            counts[g] += 1
        for i, src in enumerate(cache_of):
            if src is not None:
                if type(entry_specs[i]) is not type(entry_specs[src]):
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {src}: different kinds")
                if isinstance(entry_specs[i], PagedKVSpec) and entry_specs[i] != entry_specs[src]:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {src}: "
                                     f"{entry_specs[i]} against {entry_specs[src]}")
        self.group_keys = group_keys
        self.group_entries = counts
        if not group_keys:
            # A model without paged mixers still gets one (empty) group, so that the
            # manager, the tables and the scheduler work unchanged.
            self.group_keys = [(0, 0, 0)]
            self.group_entries = [0]
        self.manager = host.CacheManager(
            [host.GroupSpec(self.page_size, key[2]) for key in self.group_keys],
            [self.num_pages] * len(self.group_keys), self.num_slots)
        self.max_pages = [(int(max_model_len) + self.page_size - 1) // self.page_size] * len(self.group_keys)
        self.kv: List[Optional[torch.Tensor]] = []
        self.states: Dict[int, torch.Tensor] = {}
        self._entry_specs, self._cache_of = list(entry_specs), list(cache_of)
        if allocate:
            # One page and one slot more than the manager hands out: padding rows of a
            # fixed-shape (graph) batch write there.
            for (nkv, d, _w), n in zip(self.group_keys, self.group_entries):
                self.kv.append(torch.zeros((max(n, 0), 2, self.num_pages + 1, nkv, self.page_size, d),
                                           dtype=dtype, device=self.device) if n else None)
            for i, spec in enumerate(entry_specs):
                if isinstance(spec, SlotStateSpec) and cache_of[i] is None:
                    self.states[i] = torch.zeros((self.num_slots + 1,) + tuple(spec.shape), dtype=spec.dtype,
                                                 device=self.device)

    @property
    def scratch_page(self) -> int:
        return self.num_pages

    @property
    def scratch_slot(self) -> int:
        return self.num_slots

    def bytes_per_page(self) -> int:
        esz = torch.empty((), dtype=self.dtype).element_size()
        return sum(n * 2 * nkv * self.page_size * d * esz for (nkv, d, _), n in zip(self.group_keys, self.group_entries))

    @staticmethod
    def bytes_per_token(entry_specs, cache_of, dtype) -> int:
        esz = torch.empty((), dtype=dtype).element_size()
        return sum(2 * s.num_kv_heads * s.head_dim * esz for i, s in enumerate(entry_specs)
                   if isinstance(s, PagedKVSpec) and cache_of[i] is None)

    def binding(self, entry: int):
        src = self._cache_of[entry]
        owner = entry if src is None else src
        spec = self._entry_specs[owner]
        if isinstance(spec, PagedKVSpec):
            g, idx = self.entry_group[owner]
            t = self.kv[g]
            return PagedKVBinding(k=t[idx, 0], v=t[idx, 1], group=g, page_size=self.page_size,
                                  write=(src is None))
        if isinstance(spec, SlotStateSpec):
            return SlotStateBinding(state=self.states[owner], write=(src is None))
        return None

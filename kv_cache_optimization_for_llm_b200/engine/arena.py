"""The memory that a step's activations live in: allocated once, handed out again every step.

Upstream allocates every buffer of a pass once at start-up, sized by MAX_BATCH_TOKENS
(allocateDeviceBuffers, base/src/engine.cu:62-122, base/src/engine.cuh:29-74), and its two
passes write into them by name.  Here the parts of a layer are not known in advance, so the
arena is handed out by bumping an offset instead: one region that lives for the whole step
(the float32 residual, the rows picked for the head, the logits) and two regions that layers
use in turn.  A layer's results stay valid while the layer behind it runs and are overwritten
by the layer after that; nothing is ever given back to an allocator, and a step of the same
shape finds every tensor at the same address as the step before (which is also what lets a
captured graph and the steps launched around it share the memory).

A region that turns out too small (a part nobody declared widths for) gets one more block, which
it keeps; a single tensor larger than a whole region (logits for thousands of rows at once)
bypasses the arena and comes from the allocator.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

_ALIGN = 256
_ESIZE = {torch.float32: 4, torch.bfloat16: 2, torch.int32: 4, torch.float16: 2, torch.uint8: 1, torch.int64: 8}


class _Region:
    def __init__(self, nbytes: int, device):
        self.device = device
        self.capacity = max(_ALIGN, -(-int(nbytes) // _ALIGN) * _ALIGN)
        self.blocks: List[torch.Tensor] = []
        self.pads: List[int] = []       # bytes in front of each block's first aligned address
        self._add_block()
        self.block, self.offset = 0, self.pads[0]
        self.grown = 0
        self.views = {}                 # (block, offset), dtype, shape -> the tensor handed out there

    def _add_block(self) -> None:
        buf = torch.empty(self.capacity + _ALIGN, dtype=torch.uint8, device=self.device)
        self.blocks.append(buf)
        self.pads.append((-buf.data_ptr()) % _ALIGN)

    def reset(self) -> None:
        self.block, self.offset = 0, self.pads[0]

    def place(self, nbytes: int):
        """Where a run of ``nbytes`` bytes on a 256-byte boundary lies, as (block, offset), or None
        if the request is larger than the region was built for."""
        need = -(-nbytes // _ALIGN) * _ALIGN
        if need > self.capacity:
            return None
        while True:
            if self.offset + need <= self.pads[self.block] + self.capacity:
                at = (self.block, self.offset)
                self.offset += need
                return at
            self.block += 1
            if self.block == len(self.blocks):
                self._add_block()
                self.grown += 1
            self.offset = self.pads[self.block]

    def take(self, nbytes: int):
        """The run itself, as bytes."""
        at = self.place(nbytes)
        if at is None:
            return None
        return self.blocks[at[0]][at[1]:at[1] + nbytes]

    def tensor(self, shape: tuple, dtype: torch.dtype, nbytes: int):
        """A tensor of this shape and type over the next run of bytes.  Steps of one shape ask for the
        same tensors at the same places again and again: the views are kept (making one costs three
        calls into torch, which a step without a captured graph pays a hundred times over)."""
        at = self.place(nbytes)
        if at is None:
            return None
        key = (at, dtype, shape)
        t = self.views.get(key)
        if t is None:
            if len(self.views) > 8192:
                self.views.clear()
            t = self.blocks[at[0]][at[1]:at[1] + nbytes].view(dtype).view(shape)
            self.views[key] = t
        return t


class StepArena:
    def __init__(self, device, step_bytes: int, layer_bytes: int):
        self.device = torch.device(device)
        self.step = _Region(step_bytes, self.device)
        self.halves = (_Region(layer_bytes, self.device), _Region(layer_bytes, self.device))
        self.turn = 0
        self.current = self.step
        self.bypassed = 0        # tensors that were too large for a region and came from the allocator

    def begin_step(self) -> None:
        self.step.reset()
        self.turn = 0
        self.current = self.step

    def begin_layer(self) -> None:
        """The region that the layer before last used is the next layer's."""
        self.turn ^= 1
        self.current = self.halves[self.turn]
        self.current.reset()

    def end_layers(self) -> None:
        self.current = self.step

    def new(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(int(x) for x in shape)
        n = 1
        for x in shape:
            n *= x
        nbytes = n * _ESIZE[dtype]
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype, device=self.device)
        t = self.current.tensor(shape, dtype, nbytes)
        if t is None:
            self.bypassed += 1
            return torch.empty(shape, dtype=dtype, device=self.device)
        return t

    def bytes_held(self) -> int:
        return sum(b.numel() for r in (self.step, *self.halves) for b in r.blocks)

    def blocks_grown(self) -> int:
        return sum(r.grown for r in (self.step, *self.halves))

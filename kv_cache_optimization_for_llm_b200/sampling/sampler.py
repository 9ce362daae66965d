"""Chooses the next token of every request that reached the end of its known tokens."""

from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class Sampler:
    """Greedy, temperature and repetition-penalty sampling on the device
    (kernel: csrc/kernels/sampling.cu; upstream: sampleTokens, base/src/engine.cu:132-158).

    The random draw of a token is a pure function of (seed, request key, index of the
    token in its sequence).  Upstream draws the first token after a prompt and the
    first decoded token from the same counter, and shifts the counter by one after a
    recompute (paged_attention/src/engine.cu:1385,1804); here the index is the
    token's own position in every path.

    The record of tokens a request has produced (for the penalty) lives in the
    request's state slot: one row of bytes per slot, allocated at first use."""

    def __init__(self, vocab_size: int, num_slots: int, device, default_seed: int = 0,
                 out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
        """``out``: the device buffer [num_slots + 1] int32 that receives the tokens, row by row
        (the step function reads tokens that the host has not seen yet from it); its last
        entry carries ``status``, the kernels' error word, when one is given."""
        self.vocab_size, self.num_slots = int(vocab_size), int(num_slots)
        self.device = torch.device(device)
        self.default_seed = int(default_seed) & 0xFFFFFFFF
        self.mask = None
        self.status = status
        cap = self.num_slots
        self._out = out if out is not None else torch.zeros(cap + 1, dtype=torch.int32, device=self.device)
        assert self._out.numel() == cap + 1 and self._out.dtype == torch.int32
        # Staging for the per-row parameters (temperature, penalty | seed, key, pos, slot) and
        # for the tokens on their way back, twice: one set may still be in flight while the
        # next step is prepared.  Each set's event tells when its transfers are over.
        self._sets = []
        for _ in range(2):
            self._sets.append({
                "host_f": torch.zeros((2, cap), dtype=torch.float32, pin_memory=True),
                "host_u": torch.zeros((4, cap), dtype=torch.int32, pin_memory=True),
                "dev_f": torch.zeros((2, cap), dtype=torch.float32, device=self.device),
                "dev_u": torch.zeros((4, cap), dtype=torch.int32, device=self.device),
                "out_host": torch.zeros(cap + 1, dtype=torch.int32, pin_memory=True),
                "event": torch.cuda.Event(), "busy": False})
        self._turn = 0

    def _ensure_mask(self):
        if self.mask is None:
            self.mask = torch.zeros((self.num_slots, self.vocab_size), dtype=torch.uint8, device=self.device)

    def begin_request(self, slot: int, params: SamplingParams, produced: Sequence[int]) -> None:
        """Called when a request takes a slot (first admission, or again after it was
        dropped): rebuilds the slot's record from the tokens it already produced."""
        if params.repetition_penalty == 1.0:
            return
        self._ensure_mask()
        toks = torch.tensor(list(produced), dtype=torch.int32, device=self.device) if len(produced) else None
        ops.reset_mask(self.mask, slot, toks)

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], keys: Sequence[int],
               positions: Sequence[int], slots: Sequence[int]):
        """Starts the sampling of one step and the transfer of its tokens to the host;
        returns a handle for :meth:`read`.  ``logits`` [R, vocab] float32; row r belongs to
        the request with ``params[r]``, random-stream key ``keys[r]``, whose new token will
        sit at ``positions[r]``.  Token r stays in ``out[r]`` on the device until the next
        launch."""
        R = logits.shape[0]
        assert R == len(params) == len(keys) == len(positions) == len(slots) and R <= self.num_slots
        st = self._sets[self._turn]
        self._turn ^= 1
        if st["busy"]:
            st["event"].synchronize()       # the launch before last: long over, unless nobody read it
        if R == 0:
            return (st, 0)
        greedy = all(p.temperature <= 0 for p in params)
        no_pen = all(p.repetition_penalty == 1.0 for p in params)
        hf, hu = st["host_f"].numpy(), st["host_u"].numpy().view(np.uint32)
        # one assignment per row of the tables (a loop over the requests costs a microsecond per element)
        hf[0, :R] = [p.temperature for p in params]
        hf[1, :R] = [p.repetition_penalty for p in params]
        ds = self.default_seed
        hu[0, :R] = [(ds if p.seed is None else int(p.seed)) & 0xFFFFFFFF for p in params]
        hu[1, :R] = [int(k) & 0xFFFFFFFF for k in keys]
        hu[2, :R] = [int(q) & 0xFFFFFFFF for q in positions]
        hu[3, :R] = [int(q) for q in slots]
        dev_f, dev_u = st["dev_f"], st["dev_u"]
        dev_u[:, :R].copy_(st["host_u"][:, :R], non_blocking=True)
        if not (greedy and no_pen):
            dev_f[:, :R].copy_(st["host_f"][:, :R], non_blocking=True)
        if not no_pen:
            self._ensure_mask()
        ops.sample(
            logits,
            None if greedy else dev_f[0], dev_u[0], dev_u[1], dev_u[2],
            None if no_pen else dev_f[1], None if no_pen else self.mask, dev_u[3],
            out=self._out, status=self.status, status_at=self.num_slots)
        st["out_host"].copy_(self._out, non_blocking=True)
        st["event"].record()
        st["busy"] = True
        return (st, R)

    def read(self, handle):
        """Waits for a launch's tokens.  Returns (token ids, kernel status word)."""
        st, R = handle
        if R == 0:
            return [], 0
        st["event"].synchronize()
        st["busy"] = False
        vals = st["out_host"].tolist()
        return vals[:R], (vals[self.num_slots] if self.status is not None else 0)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], keys: Sequence[int],
               positions: Sequence[int], slots: Sequence[int]) -> List[int]:
        """:meth:`launch` and :meth:`read` in one; the tokens only."""
        return self.read(self.launch(logits, params, keys, positions, slots))[0]

"""Chooses the next token of every request that reached the end of its known tokens."""

from __future__ import annotations

from typing import List, Sequence

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

    def __init__(self, vocab_size: int, num_slots: int, device, default_seed: int = 0):
        self.vocab_size, self.num_slots = int(vocab_size), int(num_slots)
        self.device = torch.device(device)
        self.default_seed = int(default_seed) & 0xFFFFFFFF
        self.mask = None
        cap = self.num_slots
        # staging for the per-row parameters: temperature, penalty | seed, key, pos | slot
        self._host_f = torch.zeros((2, cap), dtype=torch.float32, pin_memory=True)
        self._host_u = torch.zeros((4, cap), dtype=torch.int32, pin_memory=True)
        self._dev_f = torch.zeros((2, cap), dtype=torch.float32, device=self.device)
        self._dev_u = torch.zeros((4, cap), dtype=torch.int32, device=self.device)
        self._out = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._out_host = torch.zeros(cap, dtype=torch.int32, pin_memory=True)

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

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], keys: Sequence[int],
               positions: Sequence[int], slots: Sequence[int]) -> List[int]:
        """``logits`` [R, vocab] float32; row r belongs to the request with ``params[r]``,
        random-stream key ``keys[r]``, whose new token will sit at ``positions[r]``."""
        R = logits.shape[0]
        assert R == len(params) == len(keys) == len(positions) == len(slots)
        if R == 0:
            return []
        greedy = all(p.temperature <= 0 for p in params)
        no_pen = all(p.repetition_penalty == 1.0 for p in params)
        hf, hu = self._host_f.numpy(), self._host_u.numpy().view(np.uint32)
        for r, p in enumerate(params):
            hf[0, r] = p.temperature
            hf[1, r] = p.repetition_penalty
            hu[0, r] = (self.default_seed if p.seed is None else int(p.seed)) & 0xFFFFFFFF
            hu[1, r] = int(keys[r]) & 0xFFFFFFFF
            hu[2, r] = int(positions[r]) & 0xFFFFFFFF
            hu[3, r] = int(slots[r])
        self._dev_u[:, :R].copy_(self._host_u[:, :R], non_blocking=True)
        if not (greedy and no_pen):
            self._dev_f[:, :R].copy_(self._host_f[:, :R], non_blocking=True)
        if not no_pen:
            self._ensure_mask()
        out = ops.sample(
            logits,
            None if greedy else self._dev_f[0], self._dev_u[0], self._dev_u[1], self._dev_u[2],
            None if no_pen else self._dev_f[1], None if no_pen else self.mask, self._dev_u[3],
            out=self._out)
        self._out_host[:R].copy_(out[:R], non_blocking=False)
        return self._out_host[:R].tolist()

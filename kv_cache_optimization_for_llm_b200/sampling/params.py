"""Per-request sampling options.

Upstream sets these for the whole engine through environment variables
(TEMPERATURE, SAMPLING_SEED, IGNORE_EOS: base/src/main.cu:52-79) and fixes the
repetition penalty at 1.15 (base/src/config.h:83); here they belong to a request,
with the same meanings."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    max_tokens: int = 16                 # output budget of the request (upstream: max_tokens on the wire)
    temperature: float = 0.0             # <= 0: greedy (upstream: TEMPERATURE unset or 0)
    seed: Optional[int] = None           # None: the engine's seed (upstream: SAMPLING_SEED)
    ignore_eos: bool = False             # keep generating through stop tokens (upstream: IGNORE_EOS=1)
    repetition_penalty: float = 1.0      # 1.0: off; upstream always applies 1.15 while decoding

    def __post_init__(self):
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.temperature < 0:
            self.temperature = 0.0       # upstream clamps a negative temperature to greedy

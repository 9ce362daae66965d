"""The Python entry point: ``LLM(model_dir).generate(prompts, SamplingParams(...))``."""

from __future__ import annotations

from typing import List, Optional, Sequence

from .config import EngineConfig
from .sampling.params import SamplingParams


class LLM:
    """A loaded model with its cache and scheduler.  Keyword arguments are the fields
    of :class:`EngineConfig` (dtype, page_size, num_pages, max_num_seqs, ...)."""

    def __init__(self, model_dir, _random_init=None, **engine_kwargs):
        from .engine.llm_engine import LLMEngine
        self.engine = LLMEngine(model_dir, EngineConfig(**engine_kwargs), random_init=_random_init)

    @classmethod
    def from_random(cls, config_dict: dict, seed: int = 0, std: float = 0.02, **engine_kwargs) -> "LLM":
        """The architecture that ``config_dict`` (a config.json) names, with random weights
        drawn on the device: matrices N(0, std), norm weights 1 + N(0, std)."""
        return cls(None, _random_init={"config": config_dict, "seed": seed, "std": std}, **engine_kwargs)

    def generate(self, prompts: Sequence[Sequence[int]], sampling=None) -> List[List[int]]:
        """``prompts``: token ids per prompt.  ``sampling``: one SamplingParams for all or
        one per prompt.  Returns the generated token ids per prompt (stop token not
        included)."""
        return self.engine.generate(prompts, sampling)


def generate(model_dir, prompts: Sequence[Sequence[int]], sampling: Optional[SamplingParams] = None,
             **engine_kwargs) -> List[List[int]]:
    return LLM(model_dir, **engine_kwargs).generate(prompts, sampling)

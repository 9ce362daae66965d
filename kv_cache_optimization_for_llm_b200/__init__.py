"""A small, whole inference engine for the Llama dense decoder on one B200.

    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams, generate
    out = generate("path/to/model", [[1, 2, 3]], SamplingParams(max_tokens=8))

Token ids in, token ids out: as upstream's engine, this one never sees text; a
tokenizer belongs to the client (base/client.py:276-304).
"""

from .config import EngineConfig
from .sampling.params import SamplingParams

__all__ = ["EngineConfig", "SamplingParams", "LLM", "generate", "write_random_model"]


def __getattr__(name):
    if name == "LLM":
        from .api import LLM
        return LLM
    if name == "generate":
        from .api import generate
        return generate
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)

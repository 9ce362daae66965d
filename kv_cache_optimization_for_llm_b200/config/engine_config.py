"""Run-time limits of the engine.

Upstream fixes these at compile time (MAX_SEQUENCES, MAX_BATCH_TOKENS, MAX_SEQ_LEN,
BLOCK_SIZE, KV_SAFETY_MARGIN_BYTES: base/src/config.h:80-136,
paged_attention/src/config.h:181-193); here they are values of one object.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = ("bfloat16", "float32")


def canonical_dtype(name: str) -> str:
    alias = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp32": "float32", "float32": "float32",
             "f32": "float32", "float": "float32"}
    try:
        return alias[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not one of {DTYPES}") from None


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"             # "bfloat16": serving precision; "float32": true 32-bit everywhere
    page_size: int = 16                 # tokens per cache page
    num_pages: Optional[int] = None     # None: from memory_fraction of the free device memory
    memory_fraction: float = 0.5
    max_num_seqs: int = 64              # requests that hold cache at once (= state slots)
    max_num_batched_tokens: int = 2048  # tokens per step
    max_model_len: Optional[int] = None  # None: the model's max_position_embeddings
    max_prefill_chunk: int = 0          # 0: only the token budget cuts a prompt
    max_portions_per_step: int = 0      # prompt portions a step may hold (0: any number).  One a step lets nearly every
                                        # step of a 1B model replay from a graph, yet measured worse under 300 short
                                        # prompts a second (21.4k against 22.4k tokens/s, first token after 266 ms
                                        # against 73 ms): the queue drains one prompt a step.  Hence off
    seed: int = 0                       # engine-wide sampling seed (upstream's SAMPLING_SEED)
    use_cuda_graphs: bool = True        # replay decode-only steps from captured graphs
    capture_graphs_at_start: bool = False  # capture every decode graph when the engine is built, not at first use
    graph_mixed_steps: Optional[bool] = None   # also replay steps of single tokens beside one short portion from graphs
                                        # (padded).  Pays when steps are bound by the host, costs when the GPU is the
                                        # bound (measured: +20 % output tokens/s at the 1B shape under a chat-like load,
                                        # -6 % at the 3B shape).  None: on for models of at most 4 GB of weights
    run_ahead: bool = True              # launch the next step before the last step's tokens reach the host
    device: str = "cuda:0"

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        if self.page_size < 1:
            raise ValueError("page_size must be >= 1")
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be >= 1")

"""This package's logits, and the plain implementation's, against what upstream's own engine
generated.  ``tests/golden/upstream_tokens_llama1b.json`` holds, for six prompts of 5 to 1000
random tokens on a Llama-3.2-1B-shaped model with random weights (seed 0), the 16 tokens that
upstream's unmodified paged engine produced greedily (made on a B200 by
``tests/golden/make_upstream_tokens.py``).  The same model is written again here from the same
seed, every prompt is followed token by token along upstream's own continuation, and at each of
the 96 places upstream's token must be the best, or all but the best, of the 128 256 under the
logits computed here (with upstream's repetition penalty of 1.15 on the tokens the request has
produced so far, as upstream applies it).  Upstream keeps its residual stream and its logits in
bfloat16, so a tie within a rounding (2^-9 of a logit) may go the other way there: its token may
be second, and its logit here may lie below the best by a few roundings, not more.  By chance a
token would be among the best two of 128 256 once in 64 000 tries."""

import json
import os
import shutil
import tempfile

import numpy as np
import pytest

import plain_llama as P

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "upstream_tokens_llama1b.json")
MAX_RANK = 2            # best, second or third of 128 256
MAX_GAP = 2e-2          # of the largest logit: some ten bfloat16 roundings


@pytest.fixture(scope="module")
def golden():
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    g = json.load(open(GOLDEN))
    d = tempfile.mkdtemp(prefix="kvb200_upstream_")
    write_random_model(d, g["config"], g["seed"], g["std"], storage_dtype=g["storage_dtype"])
    yield g, d
    shutil.rmtree(d, ignore_errors=True)


def _place(logits, toks, k, penalty):
    """Rank of upstream's k-th token under ``logits`` (0: the best) and how far below the best it lies."""
    l = P.penalise(logits, toks[:k], penalty) if k else np.asarray(logits, dtype=np.float64)
    return int((l > l[toks[k]]).sum()), float((l.max() - l[toks[k]]) / np.abs(l).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_upstreams_greedy_tokens_are_the_best_under_our_logits(golden, dtype):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    g, d = golden
    r = ModelRunner(d, EngineConfig(dtype=dtype, page_size=16, num_pages=200, max_num_seqs=2,
                                    max_num_batched_tokens=1024, max_model_len=2048, use_cuda_graphs=False))
    ranks, gaps = [], []
    for i, (prompt, toks) in enumerate(zip(g["prompts"], g["tokens"])):
        logits = r.step([StepEntry(i, prompt, 0, [len(prompt) - 1])])[0].cpu().numpy()
        for k, tok in enumerate(toks):
            rank, gap = _place(logits, toks, k, g["repetition_penalty"])
            ranks.append(rank)
            gaps.append(gap)
            assert rank <= MAX_RANK and gap < MAX_GAP, (dtype, i, k, rank, gap)
            logits = r.step([StepEntry(i, [tok], len(prompt) + k, [0])])[0].cpu().numpy()
        r.release(i)
    r.check_status()
    best = sum(x == 0 for x in ranks) / len(ranks)
    assert len(ranks) == 96 and best >= 0.9, (best, ranks)
    print(f"{dtype}: upstream's token is our best at {100 * best:.0f} % of 96 places, never below rank {max(ranks)}, "
          f"at most {max(gaps):.1e} of the largest logit below the best")


def test_upstreams_greedy_tokens_are_the_best_under_the_plain_implementation(golden):
    """The plain implementation itself (numpy, float64, whole sequences, no cache) on the shortest
    prompt followed by upstream's 16 tokens: 21 positions of the 16-layer model."""
    g, d = golden
    cfg, w = P.read_model_dir(d)
    prompt, toks = g["prompts"][0], g["tokens"][0]
    seq = prompt + toks[:-1]
    logits = P.forward(cfg, w, seq, rows=range(len(prompt) - 1, len(seq)))
    ranks = []
    for k in range(len(toks)):
        rank, gap = _place(logits[k], toks, k, g["repetition_penalty"])
        ranks.append(rank)
        assert rank <= MAX_RANK and gap < MAX_GAP, (k, rank, gap)
    assert sum(x == 0 for x in ranks) >= 14, ranks

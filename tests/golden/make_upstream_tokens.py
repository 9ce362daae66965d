"""Makes ``upstream_tokens_llama1b.json``: what upstream's own engine generates, greedily, for a
few prompts on a Llama-3.2-1B-shaped model with random weights.  Run once, by hand, on a machine
with a GPU and with upstream's paged_attention sources compiled as ``bench.py --impl reference``
compiles them (unmodified, for sm_100a, under baseline/_ref):

    python tests/golden/make_upstream_tokens.py

The model is the one ``write_random_model(LLAMA_1B, seed=0, std=0.02, "bfloat16")`` writes (the
test writes it again from the same numbers; the folder itself is 2.5 GB and is not kept).  The
engine is driven through its wire format with ``IGNORE_EOS=1`` and no ``TEMPERATURE``: greedy
decoding, with upstream's built-in repetition penalty of 1.15 on the tokens a request has
produced (paged_attention/src/kernels.cu:516-530, applied from the second generated token on:
engine.cu:1373-1390,1806-1808).  The file holds the prompts and the tokens upstream produced;
``tests/test_upstream_golden_gpu.py`` checks this package's logits against them.
"""

import json
import os
import shutil
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
}
SEED, STD, PROMPT_SEED, NEW_TOKENS = 0, 0.02, 123, 16
PROMPT_LENGTHS = [5, 33, 64, 200, 512, 1000]


def main():
    import torch
    import reference_arm as R
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    R.ensure_built()
    tmp = tempfile.mkdtemp(prefix="kvb200_golden_")
    eng = None
    try:
        model_dir = write_random_model(os.path.join(tmp, "model"), LLAMA_1B, SEED, STD, storage_dtype="bfloat16")
        rng = np.random.default_rng(PROMPT_SEED)
        prompts = [rng.integers(0, LLAMA_1B["vocab_size"], n).tolist() for n in PROMPT_LENGTHS]
        eng, pages, _held = R.start_engine_with_a_pool_that_fits(torch, str(model_dir), tmp)
        tokens = []
        for i, p in enumerate(prompts):           # one at a time: every request alone in its steps
            base = len(eng.snapshot())
            eng.send(R.request_lines([i], [p], NEW_TOKENS))
            eng.wait_for(lambda d, i=i: d.get("done") and d.get("id") == i, 300, f"generating for prompt {i}")
            tokens.append([d["tok"] for _, d in eng.snapshot()[base:] if "tok" in d and d.get("id") == i])
            assert len(tokens[-1]) == NEW_TOKENS, tokens[-1]
        out = {"config": LLAMA_1B, "seed": SEED, "std": STD, "storage_dtype": "bfloat16",
               "repetition_penalty": 1.15, "prompts": prompts, "tokens": tokens,
               "made_by": "tests/golden/make_upstream_tokens.py with upstream's paged_attention engine, unmodified, sm_100a"}
        with open(os.path.join(HERE, "upstream_tokens_llama1b.json"), "w") as f:
            json.dump(out, f)
        print("wrote", len(prompts), "prompts;", [t[:4] for t in tokens])
    finally:
        if eng is not None:
            eng.stop()
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()

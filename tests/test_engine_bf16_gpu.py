"""bfloat16 through the scheduler: the engine one step ahead, decode steps replayed from
captured graphs (3, 5 and 7 live requests pad to graphs of 4 and 8 rows), prompts in portions
beside decode tokens, a pool so small that requests are dropped and recomputed, the norm
weights folded into the products.  Compared are the logits of every sampled row, not the
tokens: at 4e-2 of the largest logit, against the plain implementation on the sequences that
the engine produced."""

import numpy as np
import pytest

import plain_llama as P
from logit_hook import LogitRecorder
from tiny_models import model_dir

pytestmark = pytest.mark.gpu

LENGTHS = [33, 70, 120, 9, 50, 64, 17]


@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
@pytest.mark.parametrize("n_reqs,num_pages,n_new", [(3, 40, 24), (5, 40, 24), (7, 18, 48)])
def test_bf16_engine_logits_with_graphs_padding_rows_and_preemption(name, n_reqs, num_pages, n_new):
    from kv_cache_optimization_for_llm_b200 import EngineConfig, SamplingParams
    from kv_cache_optimization_for_llm_b200.engine.llm_engine import LLMEngine
    mdir = model_dir(name, "bfloat16")
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(40 + n_reqs)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in LENGTHS[:n_reqs]]
    eng = LLMEngine(mdir, EngineConfig(dtype="bfloat16", page_size=16, num_pages=num_pages, max_num_seqs=8,
                                       max_num_batched_tokens=48, max_model_len=320, seed=5,
                                       use_cuda_graphs=True, run_ahead=True))
    rec = LogitRecorder(eng.runner)
    params = [SamplingParams(max_tokens=n_new, temperature=0.7, seed=300 + i, ignore_eos=True) for i in range(n_reqs)]
    ids, step = [], 0
    while len(ids) < n_reqs or eng.has_unfinished():
        if step % 2 == 0 and len(ids) < n_reqs:
            ids.append(eng.add_request(prompts[len(ids)], params[len(ids)]))
        eng.step()
        assert eng.runner.manager.check() == ""
        step += 1
        assert step < 3000
    st = eng.stats()
    assert st["free_pages"] == [num_pages]
    if n_reqs == 7:
        assert st["preemptions"] > 0, "the pool was meant to be too small"
    seqs = {rid: prompts[i] + eng.output(rid) for i, rid in enumerate(ids)}
    assert all(len(eng.output(rid)) == n_new for rid in ids)
    n, worst = rec.compare(seqs, lambda rid: P.forward(cfg, w, seqs[rid]), 4e-2, f"{name}, {n_reqs} requests")
    assert n >= n_reqs * n_new
    # decode-only steps whose number of rows is no power of two ran, each from a graph of the
    # next larger size, with padding rows
    padded = {rows for rows, single in rec.steps if single and rows & (rows - 1)}
    assert padded, rec.steps
    for rows in padded:
        bucket = next(b for b in eng.runner.graph_buckets if b >= rows)
        assert any(key[0] == bucket for key in eng.runner._graphs), (rows, list(eng.runner._graphs))
    print(f"{name}, {n_reqs} requests: {n} rows, worst relative error {worst:.3e}, preemptions {st['preemptions']}")


# head size 128 in groups of four, long enough a portion that the 128-row query tiles fill the GPU
WIDE_128 = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 600, "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 256},
    "max_position_embeddings": 1536, "tie_word_embeddings": False, "hidden_act": "silu",
}


def test_long_portion_at_head_size_128_through_the_engine():
    """bfloat16, head size 128: a portion of 1280 tokens in one step takes the warp-specialised
    tcgen05 attention (the kernel the 3B and 8B shapes read their prompts with); then a second
    portion over the cache the first left, and single tokens.  Logits against the plain
    implementation at the first row, across tile and page edges, and at the end."""
    import tempfile, shutil
    from kv_cache_optimization_for_llm_b200 import EngineConfig, ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    d = tempfile.mkdtemp(prefix="kvb200_wide128_")
    try:
        write_random_model(d, WIDE_128, seed=7, std=0.05, storage_dtype="bfloat16")
        cfg, w = P.read_model_dir(d)
        seq = np.random.default_rng(3).integers(0, 600, 1500).tolist()
        rows_a, rows_b = [0, 31, 32, 63, 64, 127, 128, 700, 1279], [0, 1, 100, 199]
        ref = P.forward(cfg, w, seq, rows=rows_a + [1280 + r for r in rows_b] + list(range(1480, 1500)))
        r = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=16, num_pages=100, max_num_seqs=2,
                                        max_num_batched_tokens=1280, max_model_len=1536, use_cuda_graphs=False))
        ops.choices.clear()
        got = [r.step([StepEntry(0, seq[:1280], 0, rows_a)]).cpu().numpy()]
        assert ops.choices["flash_attention_3"] == WIDE_128["num_hidden_layers"], dict(ops.choices)
        got.append(r.step([StepEntry(0, seq[1280:1480], 1280, rows_b)]).cpu().numpy())   # over the cache, smaller tiles
        for i in range(1480, 1500):
            got.append(r.step([StepEntry(0, [seq[i]], i, [0])]).cpu().numpy())
        r.check_status()
        got = np.concatenate(got)
        err = np.abs(got - ref).max() / np.abs(ref).max()
        assert err < 4e-2, err
        print(f"head size 128, 1280-token portion: worst relative error {err:.3e}")
    finally:
        shutil.rmtree(d)


LONG_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 515, "hidden_size": 256, "intermediate_size": 384, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "max_position_embeddings": 2304, "tie_word_embeddings": True, "hidden_act": "silu",
}


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_decoding_across_the_edge_of_a_context_class(dtype, tol):
    """Launches, captured graphs and the width of the block tables come in classes by the step's
    longest context (up to 2048 tokens, up to 8192, beyond).  Two requests decode side by side
    from graphs while the longer one grows from 2040 to 2060 tokens, across the first edge: the
    step switches graph and table width at 2049, the shorter request's logits must not notice."""
    import tempfile, shutil
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    d = tempfile.mkdtemp(prefix="kvb200_long_")
    try:
        write_random_model(d, LONG_D, seed=21, std=0.05, storage_dtype="float32" if dtype == "float32" else "bfloat16")
        cfg, w = P.read_model_dir(d)
        rng = np.random.default_rng(9)
        long_seq, short_seq = rng.integers(0, 515, 2060).tolist(), rng.integers(0, 515, 60).tolist()
        ref_long = P.forward(cfg, w, long_seq, rows=range(2039, 2060))
        ref_short = P.forward(cfg, w, short_seq, rows=range(39, 60))
        r = ModelRunner(d, EngineConfig(dtype=dtype, page_size=16, num_pages=160, max_num_seqs=2,
                                        max_num_batched_tokens=1100, max_model_len=2304, use_cuda_graphs=True))
        r.step([StepEntry(0, long_seq[:1024], 0, [])])
        out = r.step([StepEntry(0, long_seq[1024:2040], 1024, [1015]), StepEntry(1, short_seq[:40], 0, [39])]).cpu().numpy()
        worst = max(np.abs(out[0] - ref_long[0]).max() / np.abs(ref_long).max(),
                    np.abs(out[1] - ref_short[0]).max() / np.abs(ref_short).max())
        for k in range(20):          # contexts 2041 .. 2060 beside 41 .. 60
            out = r.step([StepEntry(0, [long_seq[2040 + k]], 2040 + k, [0]),
                          StepEntry(1, [short_seq[40 + k]], 40 + k, [0])]).cpu().numpy()
            worst = max(worst, np.abs(out[0] - ref_long[1 + k]).max() / np.abs(ref_long).max(),
                        np.abs(out[1] - ref_short[1 + k]).max() / np.abs(ref_short).max())
        r.check_status()
        classes = sorted(key[1] for key in r._graphs)
        assert classes == [4, 8], classes          # both sides of the edge ran, each from a graph of its own
        assert worst < tol, worst
    finally:
        shutil.rmtree(d)

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

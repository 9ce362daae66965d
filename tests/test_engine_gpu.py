"""The engine end to end against the plain implementation: greedy generation through
the Python entry point, sampling with per-request seeds, staggered arrivals that put
prompt portions beside decode tokens, a pool so small that requests are dropped and
recomputed, long decoding, and the first tokens of a sequence."""

import numpy as np
import pytest

import plain_llama as P
from tiny_models import CONFIGS, model_dir

pytestmark = pytest.mark.gpu


def _prompts(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"] - 2, size=n).tolist() for n in lengths]


@pytest.mark.parametrize("name,lengths,page_size", [("tiny_a", [5, 11, 17], 4), ("tiny_c", [3, 20, 9], 16)])
def test_greedy_generation_through_entry_point(name, lengths, page_size):
    """float32, greedy: the generated ids equal the plain implementation's."""
    from kv_cache_optimization_for_llm_b200 import SamplingParams, generate
    mdir = model_dir(name, "float32")
    cfg, w = P.read_model_dir(mdir)
    prompts = _prompts(cfg, lengths, 7)
    got = generate(mdir, prompts, SamplingParams(max_tokens=8, ignore_eos=True), dtype="float32",
                   page_size=page_size, num_pages=64, max_num_seqs=4, max_num_batched_tokens=32)
    for p, g in zip(prompts, got):
        assert g == P.generate(cfg, w, p, 8)


def test_greedy_same_tokens_however_scheduled():
    """float32, greedy: whole prompts, a budget of 3 tokens per step, and one request
    at a time all give the same ids."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompts = _prompts(cfg, [5, 11, 17], 11)
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    ref = [P.generate(cfg, w, p, 8) for p in prompts]
    for kw in (dict(max_num_batched_tokens=64), dict(max_num_batched_tokens=4, max_prefill_chunk=3),
               dict(max_num_seqs=1, max_num_batched_tokens=64)):
        llm = LLM(mdir, dtype="float32", page_size=4, num_pages=40, **{"max_num_seqs": 4, **kw})
        assert llm.generate(prompts, sp) == ref, kw
        assert llm.engine.runner.manager.check() == ""
        assert llm.engine.runner.manager.free_pages(0) == 40


def test_stop_token_ends_request_and_is_not_returned():
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompt = _prompts(cfg, [9], 3)[0]
    free_run = P.generate(cfg, w, prompt, 12)
    # Declare the 5th generated token a stop token through a copy of the model folder.
    import json, os, shutil, tempfile
    d = tempfile.mkdtemp(prefix="kvb200_eos_")
    shutil.copy(os.path.join(mdir, "model.safetensors"), d)
    c = dict(cfg)
    c["eos_token_id"] = int(free_run[4])
    json.dump(c, open(os.path.join(d, "config.json"), "w"))
    cut = free_run.index(free_run[4])
    llm = LLM(d, dtype="float32", page_size=4, num_pages=40, max_num_seqs=2)
    assert llm.generate([prompt], SamplingParams(max_tokens=12)) == [free_run[:cut]]
    assert llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True)) == [free_run]


def test_temperature_sampling_with_preemption_tiny_b():
    """float32, temperature 0.7 with per-request seeds, five prompts arriving two steps
    apart so that prompt portions share steps with decode tokens, 60 new tokens each, in 13
    pages of 16 tokens (all five together grow to 36): the longest prompt waits until its pages
    are free, and as the running requests grow the latest of them is dropped and recomputed.
    Every request's tokens still equal the plain implementation's, which knows no cache at all."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig, SamplingParams
    from kv_cache_optimization_for_llm_b200.engine.llm_engine import LLMEngine
    mdir = model_dir("tiny_b", "float32")
    cfg, w = P.read_model_dir(mdir)
    lengths = [1, 9, 33, 70, 120]
    prompts = _prompts(cfg, lengths, 5)
    n_new = 60
    eng = LLMEngine(mdir, EngineConfig(dtype="float32", page_size=16, num_pages=13, max_num_seqs=5,
                                       max_num_batched_tokens=48, max_model_len=256, seed=99))
    params = [SamplingParams(max_tokens=n_new, temperature=0.7, seed=1000 + i, ignore_eos=True) for i in range(5)]
    ids, step = [], 0
    while len(ids) < 5 or eng.has_unfinished():
        if step % 2 == 0 and len(ids) < 5:
            ids.append(eng.add_request(prompts[len(ids)], params[len(ids)]))
        eng.step()
        assert eng.runner.manager.check() == ""
        step += 1
        assert step < 2000
    st = eng.stats()
    assert st["preemptions"] > 0, "the pool was meant to be too small"
    assert st["free_pages"] == [13]
    for i, rid in enumerate(ids):
        ref = P.generate(cfg, w, prompts[i], n_new, temperature=0.7, seed=1000 + i, key=rid)
        assert eng.output(rid) == ref, f"request {i} (preempted {eng.preemptions_of(rid)} times)"


def test_repetition_penalty_matches_plain():
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompt = _prompts(cfg, [6], 21)[0]
    llm = LLM(mdir, dtype="float32", page_size=4, num_pages=40, max_num_seqs=2)
    got = llm.generate([prompt], SamplingParams(max_tokens=20, ignore_eos=True, repetition_penalty=1.15))[0]
    assert got == P.generate(cfg, w, prompt, 20, penalty=1.15)
    plain = llm.generate([prompt], SamplingParams(max_tokens=20, ignore_eos=True))[0]
    assert plain == P.generate(cfg, w, prompt, 20)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_long_decoding_and_first_tokens(dtype, tol):
    """A 3-token prompt, then 200 tokens one by one (tiny_b, 256 positions): logits at
    every step against the plain implementation, the very first positions included."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    mdir = model_dir("tiny_b", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(mdir)
    seq = _prompts(cfg, [203], 17)[0]
    ref = P.forward(cfg, w, seq)
    r = ModelRunner(mdir, EngineConfig(dtype=dtype, page_size=16, num_pages=13, max_num_seqs=2,
                                       max_num_batched_tokens=16, max_model_len=208))
    scale = np.abs(ref).max()
    got = r.step([StepEntry(0, seq[:1], 0, [0])]).cpu().numpy()          # a request of one token
    assert np.abs(got - ref[0:1]).max() / scale < tol
    got = r.step([StepEntry(0, seq[1:3], 1, [0, 1])]).cpu().numpy()
    assert np.abs(got - ref[1:3]).max() / scale < tol
    worst = 0.0
    for i in range(3, len(seq)):
        got = r.step([StepEntry(0, [seq[i]], i, [0])]).cpu().numpy()
        worst = max(worst, np.abs(got - ref[i:i + 1]).max() / scale)
    r.check_status()
    assert worst < tol, worst


@pytest.mark.parametrize("name", ["tiny_d", "tiny_e"])
def test_norm_weights_far_from_one(name):
    """bfloat16: the layers' norm weights are multiplied into the matrices behind them and,
    for steps of few tokens, the add and the norm happen inside the products.  With norm
    weights spread over 0.25 .. 4 a weight that went missing, was applied twice or landed on
    the wrong matrix shows at once: in one step of many tokens (separate norm kernel), in
    steps of a few tokens and token by token, against the plain implementation."""
    import json, os, shutil, tempfile
    import torch
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.weights.safetensors_io import read_tensors, write_tensors
    src = model_dir(name, "bfloat16")
    d = tempfile.mkdtemp(prefix="kvb200_norms_")
    try:
        shutil.copy(os.path.join(src, "config.json"), d)
        tensors = read_tensors(os.path.join(src, "model.safetensors"))
        g = torch.Generator().manual_seed(5)
        for k, t in tensors.items():
            if "norm" in k:
                tensors[k] = (2.0 ** (4 * torch.rand(t.shape, generator=g) - 2)).to(t.dtype)
        write_tensors(os.path.join(d, "model.safetensors"), tensors)
        cfg, w = P.read_model_dir(d)
        seq = _prompts(cfg, [70], 23)[0]
        ref = P.forward(cfg, w, seq)
        scale = np.abs(ref).max()
        r = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=16, num_pages=12, max_num_seqs=2,
                                        max_num_batched_tokens=64, max_model_len=96))
        got = [r.step([StepEntry(0, seq[:34], 0, list(range(34)))]).cpu().numpy()]      # many rows: library product
        got.append(r.step([StepEntry(0, seq[34:58], 34, list(range(24)))]).cpu().numpy())  # 24 rows: folded
        got.append(r.step([StepEntry(0, seq[58:64], 58, list(range(6)))]).cpu().numpy())   # 6 rows: folded
        for i in range(64, 70):
            got.append(r.step([StepEntry(0, [seq[i]], i, [0])]).cpu().numpy())
        r.check_status()
        got = np.concatenate(got)
        assert np.abs(got - ref).max() / scale < 4e-2
    finally:
        shutil.rmtree(d)


def test_running_ahead_changes_no_token():
    """The engine launches a step before the tokens of the step before it have reached the
    host.  With stop tokens (whose request has one more token computed for nothing), a pool
    that forces requests out and back in, and a request withdrawn while a step with it is on
    the device: the same tokens as when it waits after every step, and as the plain
    implementation; no page lost."""
    import json, os, shutil, tempfile
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompts = _prompts(cfg, [5, 30, 17, 9], 31)
    free = [P.generate(cfg, w, p, 32) for p in prompts]
    d = tempfile.mkdtemp(prefix="kvb200_ahead_")
    try:
        shutil.copy(os.path.join(mdir, "model.safetensors"), d)
        c = dict(cfg)
        c["eos_token_id"] = [int(free[0][6]), int(free[2][15])]       # both stop somewhere in the middle
        json.dump(c, open(os.path.join(d, "config.json"), "w"))
        _, w2 = P.read_model_dir(d)
        ref = [P.generate(c, w2, p, 32, eos=c["eos_token_id"]) for p in prompts]
        assert any(len(r) < 32 for r in ref)
        outs = {}
        for ahead in (False, True):
            llm = LLM(d, dtype="float32", page_size=4, num_pages=21, max_num_seqs=4, max_num_batched_tokens=16,
                      run_ahead=ahead)
            outs[ahead] = llm.generate(prompts, SamplingParams(max_tokens=32))
            assert llm.engine.stats()["preemptions"] > 0
            assert llm.engine.runner.manager.check() == "" and llm.engine.runner.manager.free_pages(0) == 21
        assert outs[True] == outs[False] == ref
        # withdrawn in flight
        llm = LLM(d, dtype="float32", page_size=4, num_pages=40, max_num_seqs=4, run_ahead=True)
        eng = llm.engine
        ids = [eng.add_request(p, SamplingParams(max_tokens=32)) for p in prompts[:2]]
        got = {i: [] for i in ids}
        for _ in range(4):
            for ev in eng.step():
                if ev.token is not None:
                    got[ev.request_id].append(ev.token)
        eng.abort(ids[0])
        while eng.has_unfinished():
            for ev in eng.step():
                assert ev.request_id != ids[0]
                if ev.token is not None:
                    got[ev.request_id].append(ev.token)
        assert got[ids[1]] == ref[1] and got[ids[0]] == ref[0][:len(got[ids[0]])]
        assert eng.runner.manager.check() == "" and eng.runner.manager.free_pages(0) == 40
    finally:
        shutil.rmtree(d)


def test_random_workload_ahead_and_waiting_agree():
    """120 requests with random prompt lengths, budgets, temperatures, seeds, penalties and
    arrival gaps, in a pool small enough to drop and recompute some: the engine one step
    ahead produces the tokens of the engine that waits after every step, and every tenth
    request's are those of the plain implementation (float32)."""
    import random
    from kv_cache_optimization_for_llm_b200 import EngineConfig, SamplingParams
    from kv_cache_optimization_for_llm_b200.engine.llm_engine import LLMEngine
    mdir = model_dir("tiny_b", "float32")
    cfg, w = P.read_model_dir(mdir)
    rng = random.Random(7)
    reqs = []
    for i in range(120):
        prompt = [rng.randrange(cfg["vocab_size"] - 2) for _ in range(rng.choice([1, 2, 3, 5, 8, 13, 21, 34, 55, 80]))]
        sp = SamplingParams(max_tokens=rng.choice([1, 2, 4, 9, 17, 30]), temperature=rng.choice([0.0, 0.0, 0.7, 1.3]),
                            seed=rng.randrange(1000), ignore_eos=True, repetition_penalty=rng.choice([1.0, 1.0, 1.15]))
        reqs.append((prompt, sp, rng.randrange(0, 3)))        # tokens, sampling, steps until the next arrival

    def run(run_ahead):
        eng = LLMEngine(mdir, EngineConfig(dtype="float32", page_size=4, num_pages=50, max_num_seqs=6,
                                           max_num_batched_tokens=24, max_model_len=128, run_ahead=run_ahead))
        out, waiting, gap, steps = {}, list(enumerate(reqs)), 0, 0
        while waiting or eng.has_unfinished():
            while waiting and gap <= 0:
                i, (prompt, sp, gap) = waiting.pop(0)
                eng.add_request(prompt, sp, request_id=i)
                out[i] = []
            gap -= 1
            for ev in eng.step():
                if ev.token is not None:
                    out[ev.request_id].append(ev.token)
            steps += 1
            assert steps < 20000
        assert eng.stats()["preemptions"] > 0
        assert eng.runner.manager.check() == "" and eng.runner.manager.free_pages(0) == 50
        return out

    ahead, waited = run(True), run(False)
    assert ahead == waited
    for i in range(0, len(reqs), 10):
        prompt, sp, _ = reqs[i]
        assert ahead[i] == P.generate(cfg, w, prompt, sp.max_tokens, temperature=sp.temperature, seed=sp.seed, key=i,
                                      penalty=sp.repetition_penalty), i


@pytest.mark.parametrize("mode", ["off", "auto", "all", "folded"])
def test_long_portion_through_the_products_for_many_rows(mode, monkeypatch):
    """bfloat16, a portion of 200 tokens in one step (tiny_b): with the library products, with
    this package's tcgen05 kernel for the gate|up product only, with it for every product, and with the
    residual add and the norm folded into its products; the logits at the first, the 128th, the 129th and the last place against the plain implementation."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig, ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    # "folded": also the residual add and the norm inside the products, as for steps of few rows
    monkeypatch.setattr(ops, "WIDE", "auto" if mode == "folded" else mode)
    monkeypatch.setattr(ops, "WIDE_FUSED_MIN_ROWS", 128 if mode == "folded" else 0)
    mdir = model_dir("tiny_b", "bfloat16")
    cfg, w = P.read_model_dir(mdir)
    seq = _prompts(cfg, [203], 23)[0]
    ref = P.forward(cfg, w, seq)
    r = ModelRunner(mdir, EngineConfig(dtype="bfloat16", page_size=16, num_pages=13, max_num_seqs=2,
                                       max_num_batched_tokens=256, max_model_len=208))
    before = ops.launch_count
    want = [0, 127, 128, 199]
    got = r.step([StepEntry(0, seq[:200], 0, want)]).cpu().numpy()
    r.check_status()
    assert np.abs(got - ref[want]).max() / np.abs(ref).max() < 4e-2
    if mode != "off":
        assert "gemm_bf16_wide" in ops.loaded_libraries()
    # the rest one by one, from the cache that the long portion left
    for i in range(200, 203):
        got = r.step([StepEntry(0, [seq[i]], i, [0])]).cpu().numpy()
        assert np.abs(got - ref[i:i + 1]).max() / np.abs(ref).max() < 4e-2
    assert ops.launch_count > before


def test_graphs_captured_when_the_engine_is_built():
    """``capture_graphs_at_start``: every decode graph (each batch-size bucket, each class of
    context length that ``max_model_len`` allows) is captured on dummy rows before any request;
    generation then captures nothing more and produces the plain implementation's tokens."""
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompts = _prompts(cfg, [5, 11, 17, 3, 8], 41)
    llm = LLM(mdir, dtype="float32", page_size=4, num_pages=64, max_num_seqs=6, max_num_batched_tokens=32,
              capture_graphs_at_start=True)
    r = llm.engine.runner
    assert r.graph_buckets == [1, 2, 4, 6] and sorted(r._graphs) == [(1, 4), (2, 4), (4, 4), (6, 4)]   # tiny_a: 128 positions, one class
    assert int(r.status.item()) == 0 and r.manager.check() == "" and r.manager.free_pages(0) == 64
    got = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert len([k for k in r._graphs if k[0] != "portion"]) == 4      # no decode graph was captured on the way
    for p, g in zip(prompts, got):
        assert g == P.generate(cfg, w, p, 8)


def test_capture_is_safe_from_the_garbage_collector():
    """An engine that is gone but still waits for the collector (it sits in a reference cycle) holds
    captured graphs; destroying them is refused while another stream is capturing, and the refusal
    would end that capture.  The runner keeps the collector out of its captures: here the first
    engine becomes garbage, and enough containers are made for the collector to run, in the middle
    of the second engine's first captured forward pass."""
    import gc
    import torch
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    prompts = _prompts(cfg, [5, 9], 43)
    kw = dict(dtype="float32", page_size=4, num_pages=64, max_num_seqs=4, max_num_batched_tokens=32)
    first = LLM(mdir, capture_graphs_at_start=True, **kw)
    assert len(first.engine.runner._graphs) > 0
    first.cycle = first                        # only the collector can free it
    held = [first]
    del first
    second = LLM(mdir, **kw)                   # captures at first use, during generation
    model = second.engine.runner.model
    inner, seen = model.forward, []

    def forward(batch, cache, arena=None):
        if torch.cuda.is_current_stream_capturing() and held:
            held.clear()
            seen.append(gc.isenabled())
            _ = [[] for _ in range(5000)]      # the collector's threshold is passed many times over
        return inner(batch, cache, arena)
    model.forward = forward
    got = second.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    assert seen == [False] and len(second.engine.runner._graphs) > 0
    assert gc.isenabled()
    for p_, g in zip(prompts, got):
        assert g == P.generate(cfg, w, p_, 6)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_a_lone_portion_is_padded_and_replayed_from_a_graph(dtype, tol):
    """A step that is one request's portion of up to 512 tokens is padded with dummy tokens to a
    fixed length and replayed from a captured graph.  The dummy tokens sit behind the run: their
    keys and values go into the rest of the request's last page and into the scratch page, and the
    tokens that follow (another portion, then single tokens) overwrite or never see them."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig, ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    name = "tiny_d" if dtype == "bfloat16" else "tiny_b"
    mdir = model_dir(name, dtype)
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(5)
    seq = rng.integers(0, cfg["vocab_size"], 60).tolist()
    ref = P.forward(cfg, w, seq)
    r = ModelRunner(mdir, EngineConfig(dtype=dtype, page_size=4, num_pages=40, max_num_seqs=4, max_num_batched_tokens=64,
                                       max_model_len=120, use_cuda_graphs=True))

    def close(got, rows):
        assert np.abs(got.cpu().numpy() - ref[rows]).max() / np.abs(ref).max() < tol

    close(r.step([StepEntry(1, seq[:37], 0, [36])]), [36])          # 37 tokens as 64: 27 dummies behind them
    assert [k for k in r._graphs if k[0] == "portion"] == [("portion", 64, (30,))]
    close(r.step([StepEntry(1, seq[37:42], 37, [4])]), [41])        # 5 tokens as 16, over the first dummies' places
    before = ops.launch_count
    close(r.step([StepEntry(2, seq[:40], 0, [39])]), [39])          # another request, the same graph again
    assert ops.launch_count == before and len([k for k in r._graphs if k[0] == "portion"]) == 2
    for i in range(42, 46):                                          # single tokens behind the portions
        close(r.step([StepEntry(1, [seq[i]], i, [0])]), [i])
    assert r.step([StepEntry(2, seq[40:60], 40, [])]).shape[0] == 0   # nothing wanted: nothing comes back
    close(r.step([StepEntry(2, [7], 60, [0]), StepEntry(1, [seq[46]], 46, [0])])[1:], [46])
    r.check_status()
    assert r.manager.check() == ""


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_single_tokens_beside_one_portion_replay_from_a_graph(dtype, tol):
    """Decoding requests beside one short portion: the requests padded with dummy requests, the
    portion with dummy tokens, the step replayed from a graph; the logits come back in the order
    of the entries, whichever of them want any, and a second step of the same shape launches nothing."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig, ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    name = "tiny_d" if dtype == "bfloat16" else "tiny_b"
    mdir = model_dir(name, dtype)
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(9)
    seqs = {i: rng.integers(0, cfg["vocab_size"], n).tolist() for i, n in ((1, 30), (2, 45), (3, 21), (4, 50), (5, 33))}
    refs = {i: P.forward(cfg, w, s) for i, s in seqs.items()}
    scale = max(np.abs(r).max() for r in refs.values())
    r = ModelRunner(mdir, EngineConfig(dtype=dtype, page_size=4, num_pages=80, max_num_seqs=6, max_num_batched_tokens=64,
                                       max_model_len=120, use_cuda_graphs=True, graph_mixed_steps=True))

    def close(got, want):          # want: [(request, position)]
        got = got.cpu().numpy()
        assert got.shape[0] == len(want)
        for row, (i, pos) in zip(got, want):
            assert np.abs(row - refs[i][pos]).max() / scale < tol, (i, pos)

    for i in (1, 2, 3):            # three requests up to their last token but two
        r.step([StepEntry(i, seqs[i][:-2], 0, [])])
    n = {i: len(seqs[i]) - 2 for i in (1, 2, 3)}
    # two decoding requests around a 20-token portion of a fourth: 2 -> 2 requests, 20 -> 32 tokens
    got = r.step([StepEntry(1, [seqs[1][n[1]]], n[1], [0]), StepEntry(4, seqs[4][:20], 0, [19]),
                  StepEntry(2, [seqs[2][n[2]]], n[2], [0])])
    close(got, [(1, n[1]), (4, 19), (2, n[2])])
    assert [k for k in r._graphs if k[0] == "mixed"] == [("mixed", 2, 32, (30,))]
    n[1] += 1; n[2] += 1
    # three decoding requests (a bucket of four) beside the next portion; one of them wants nothing
    got = r.step([StepEntry(4, seqs[4][20:50], 20, [29]), StepEntry(3, [seqs[3][n[3]]], n[3], [0]),
                  StepEntry(1, [seqs[1][n[1]]], n[1], []), StepEntry(2, [seqs[2][n[2]]], n[2], [0])])
    close(got, [(4, 49), (3, n[3]), (2, n[2])])
    n[1] += 1; n[2] += 1; n[3] += 1
    # the same shape again (one request done: two decoding, bucket of two, 32 tokens): nothing is launched
    r.release(1); r.release(2)
    before = ops.launch_count
    got = r.step([StepEntry(3, [seqs[3][n[3]]], n[3], [0]), StepEntry(5, seqs[5][:31], 0, []), StepEntry(4, [7], 50, [])])
    close(got, [(3, n[3])])
    assert ops.launch_count == before and len([k for k in r._graphs if k[0] == "mixed"]) == 2
    r.check_status()
    assert r.manager.check() == ""

"""Logits at the widths of Llama-3.2-1B against the plain implementation, through the
engine's own step function, on the paths that the benchmark times.

The model has every size of Llama-3.2-1B (hidden 2048, 32 query heads over 8 key/value
heads of size 64, feed-forward 8192, vocabulary 128 256, llama3 rotary scaling, tied head)
but LAYERS = 2 of its FULL_LAYERS = 16 layers, so that the plain implementation stays within
a minute; the kernels' launches depend on the widths, not on the depth.  Weights are stored
in bfloat16 and read by both precisions, so one set of plain logits serves both.

Covered: one 2048-token portion in a step (the warp-specialised tcgen05 attention, the
tcgen05 product for many rows with its SiLU epilogue, the head on chosen rows), the same
prompt in portions down to two tokens (the product for few rows with K split over a
cluster at N = 2048, K = 8192, the folded norms), eight requests decoding beside each other
from 512-token prompts, and 40 and 64 requests decoding from a captured graph (library
products between 33 and 127 rows, padding rows of the graph's fixed shape)."""

import shutil
import tempfile

import numpy as np
import pytest

import plain_llama as P

pytestmark = pytest.mark.gpu

FULL_LAYERS = 16
LAYERS = 2
CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": LAYERS,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
}
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
PORTIONS = [7, 2, 13, 3, 2, 5, 2, 31, 2, 4, 16, 2, 9, 64, 2, 33, 130, 2]

_state = {}


@pytest.fixture(scope="module")
def model():
    from kv_cache_optimization_for_llm_b200.weights import write_random_model
    d = tempfile.mkdtemp(prefix="kvb200_1bwide_")
    write_random_model(d, CFG, seed=0, std=0.02, storage_dtype="bfloat16")
    cfg, w = P.read_model_dir(d)
    yield d, cfg, w
    _state.clear()
    shutil.rmtree(d, ignore_errors=True)


def _runner(model_dir, dtype):
    """One runner per precision for the whole file (graphs on: steps of single tokens replay
    from a captured graph, every other step runs as launched)."""
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    key = ("runner", dtype)
    if key not in _state:
        _state[key] = ModelRunner(model_dir, EngineConfig(
            dtype=dtype, page_size=16, num_pages=900, max_num_seqs=64, max_num_batched_tokens=2048,
            max_model_len=4096, use_cuda_graphs=True))
    return _state[key]


def _ref(name, cfg, w, seq, rows):
    key = ("ref", name)
    if key not in _state:
        _state[key] = P.forward(cfg, w, seq, rows=rows)
    return _state[key]


def _check(got, ref, dtype, what):
    err = np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max()
    assert err < TOL[dtype], f"{what}: relative error {err:.3e} (limit {TOL[dtype]:.0e})"
    return err


def _long_prompt():
    return np.random.default_rng(11).integers(0, CFG["vocab_size"], 2048).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_2048_token_portion(model, dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    mdir, cfg, w = model
    seq = _long_prompt()
    rows = [0, 127, 128, 1000, 2047]
    all_rows = sorted(set(rows) | set(_portion_rows()))     # one plain pass serves the test below as well
    ref = _ref("long", cfg, w, seq, all_rows)
    pick = [all_rows.index(r) for r in rows]
    r = _runner(mdir, dtype)
    ops.choices.clear()
    got = r.step([StepEntry(1, seq, 0, rows)]).cpu().numpy()
    r.check_status()
    r.release(1)
    assert got.shape == (len(rows), CFG["vocab_size"])
    err = _check(got, ref[pick], dtype, "2048 tokens in one step")
    if dtype == "bfloat16":
        # the kernels the benchmark's prefill point runs on
        assert ops.choices["flash_attention_3"] == LAYERS, dict(ops.choices)
        assert ops.choices["gemm_wide"] >= LAYERS, dict(ops.choices)
    else:
        assert ops.choices["sgemm_nt"] > 0 and ops.choices["library_product"] == 0, dict(ops.choices)
    print(f"2048-token step, {dtype}: relative error {err:.3e}")
    assert r.manager.check() == ""
    # the same step once more, now warm: it asks the allocator for nothing
    import torch
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    again = r.step([StepEntry(3, seq, 0, rows)])
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    assert r.arena.blocks_grown() == 0 and r.arena.bypassed == 0
    _check(again.cpu().numpy(), ref[pick], dtype, "2048 tokens in one step, again")
    r.release(3)


def _portion_spans():
    spans, i, k = [], 0, 0
    while i < 2048:
        s = min(PORTIONS[k % len(PORTIONS)], 2048 - i)
        if 2048 - i - s == 1:
            s += 1
        spans.append((i, i + s))
        i += s
        k += 1
    return spans


def _portion_rows():
    return [b - 1 for _, b in _portion_spans()]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_same_prompt_in_portions_down_to_two_tokens(model, dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    mdir, cfg, w = model
    seq = _long_prompt()
    all_rows = sorted(set([0, 127, 128, 1000, 2047]) | set(_portion_rows()))
    ref = _ref("long", cfg, w, seq, all_rows)
    r = _runner(mdir, dtype)
    ops.choices.clear()
    worst = 0.0
    for a, b in _portion_spans():
        got = r.step([StepEntry(2, seq[a:b], a, [b - a - 1])]).cpu().numpy()
        worst = max(worst, _check(got, ref[all_rows.index(b - 1)][None, :], dtype, f"portion {a}:{b}"))
    r.check_status()
    r.release(2)
    if dtype == "bfloat16":
        assert ops.choices["gemm_skinny_fused"] > 0 and ops.choices["gemm_wide"] > 0, dict(ops.choices)
    print(f"portions, {dtype}: worst relative error {worst:.3e}")
    assert r.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eight_requests_decode_beside_each_other_from_512_token_prompts(model, dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    mdir, cfg, w = model
    rng = np.random.default_rng(12)
    n_prompt, n_new = 512, 8
    seqs = [rng.integers(0, CFG["vocab_size"], n_prompt + n_new).tolist() for _ in range(8)]
    rows = list(range(n_prompt - 1, n_prompt + n_new))
    refs = [_ref(f"eight{i}", cfg, w, s, rows) for i, s in enumerate(seqs)]
    r = _runner(mdir, dtype)
    ops.choices.clear()
    # four prompts to a step (2048 tokens): runs of several requests in one attention launch
    for lo in (0, 4):
        got = r.step([StepEntry(100 + i, seqs[i][:n_prompt], 0, [n_prompt - 1]) for i in range(lo, lo + 4)])
        _check(got.cpu().numpy(), np.stack([refs[i][0] for i in range(lo, lo + 4)]), dtype, f"prompts {lo}..{lo + 3}")
    worst = 0.0
    for k in range(n_new):
        got = r.step([StepEntry(100 + i, [seqs[i][n_prompt + k]], n_prompt + k, [0]) for i in range(8)])
        worst = max(worst, _check(got.cpu().numpy(), np.stack([refs[i][1 + k] for i in range(8)]), dtype,
                                  f"decode step {k}"))
    r.check_status()
    assert any(key[0] == 8 for key in r._graphs), "the decode steps were meant to replay a graph of 8 rows"
    if dtype == "bfloat16":
        assert ops.choices["decode_attention_mma"] > 0 and ops.choices["gemm_skinny_fused"] > 0, dict(ops.choices)
    for i in range(8):
        r.release(100 + i)
    print(f"8 requests, {dtype}: worst relative error {worst:.3e}")
    assert r.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_reqs", [40, 64])
def test_many_requests_decode_from_a_graph(model, dtype, n_reqs):
    """33 to 64 rows of single tokens: the graph of 64 rows (padding rows for 40), products of the
    library between 33 and 127 rows in bfloat16, one attention block per (request, kv head)."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    mdir, cfg, w = model
    rng = np.random.default_rng(13)
    n_new = 4
    lengths = rng.integers(40, 121, 64).tolist()
    seqs = [rng.integers(0, CFG["vocab_size"], n).tolist() for n in lengths]
    refs = [_ref(f"many{i}", cfg, w, s, list(range(len(s) - n_new - 1, len(s)))) for i, s in enumerate(seqs[:n_reqs])]
    r = _runner(mdir, dtype)
    base = 1000 * n_reqs
    pending = list(range(n_reqs))
    while pending:                      # prompts, as many to a step as 2048 tokens hold
        take, total = [], 0
        while pending and total + lengths[pending[0]] - n_new <= 2048:
            total += lengths[pending[0]] - n_new
            take.append(pending.pop(0))
        got = r.step([StepEntry(base + i, seqs[i][:lengths[i] - n_new], 0, [lengths[i] - n_new - 1]) for i in take])
        _check(got.cpu().numpy(), np.stack([refs[i][0] for i in take]), dtype, f"prompts {take[0]}..{take[-1]}")
    worst = 0.0
    for k in range(n_new):
        entries = [StepEntry(base + i, [seqs[i][lengths[i] - n_new + k]], lengths[i] - n_new + k, [0])
                   for i in range(n_reqs)]
        got = r.step(entries).cpu().numpy()
        worst = max(worst, _check(got, np.stack([refs[i][1 + k] for i in range(n_reqs)]), dtype, f"decode step {k}"))
    r.check_status()
    assert any(key[0] == 64 for key in r._graphs), "the decode steps were meant to replay the graph of 64 rows"
    if dtype == "bfloat16":
        # counted when the graph was captured, which an earlier test of this file may have done
        assert ops.choices["decode_attention_mma"] > 0 and ops.choices["library_product"] > 0, dict(ops.choices)
    for i in range(n_reqs):
        r.release(base + i)
    print(f"{n_reqs} requests, {dtype}: worst relative error {worst:.3e}")
    assert r.manager.check() == ""


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_tokens_beside_a_portion_take_the_decode_kernel(model, dtype):
    """A step that mixes decoding requests with a prompt portion, the entries given in an order that
    interleaves them: the batch puts the single tokens first, their attention runs in the one-launch
    kernel of decode steps, the portion's in the kernels for runs, and every logit comes back in the
    caller's order and agrees with the plain implementation."""
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    mdir, cfg, w = model
    rng = np.random.default_rng(23)
    seqs = {i: rng.integers(0, CFG["vocab_size"], n).tolist() for i, n in ((30, 140), (31, 300), (32, 75), (33, 400))}
    refs = {i: P.forward(cfg, w, s, rows=[len(s) - 2, len(s) - 1] if i != 33 else [199, 399]) for i, s in seqs.items()}
    r = _runner(mdir, dtype)
    # the three decoding requests: all but their last token as one portion each
    for i in (30, 31, 32):
        r.step([StepEntry(i, seqs[i][:-1], 0, [len(seqs[i]) - 2])])
    r.step([StepEntry(33, seqs[33][:200], 0, [199])])
    ops.choices.clear()
    got = r.step([StepEntry(30, [seqs[30][-1]], 139, [0]), StepEntry(33, seqs[33][200:], 200, [199]),
                  StepEntry(31, [seqs[31][-1]], 299, [0]), StepEntry(32, [seqs[32][-1]], 74, [0])]).cpu().numpy()
    r.check_status()
    for row, (i, ref_row) in enumerate(((30, 1), (33, 1), (31, 1), (32, 1))):
        _check(got[row:row + 1], refs[i][ref_row][None, :], dtype, f"request {i} in the mixed step")
    if dtype == "bfloat16":
        # once per layer when the step is launched, twice (warm-up and capture) when it is replayed from a graph
        flash = sum(ops.choices[f"flash_attention_{k}"] for k in range(4))
        assert ops.choices["decode_attention_mma"] == flash and flash in (LAYERS, 2 * LAYERS), dict(ops.choices)
    for i in seqs:
        r.release(i)
    assert r.manager.check() == ""

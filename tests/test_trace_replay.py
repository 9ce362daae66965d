"""Replays the same requests through bin/trace_run in every way of cutting them and
compares all logits with the plain implementation: whole; most in one step and the
last 32 tokens one by one; portions of changing size down to two tokens; and mixed,
up to four live requests with so few pages that they are used again."""

import numpy as np
import pytest

import plain_llama as P
from tiny_models import CONFIGS, model_dir
from trace_driver import TraceRun, ceil64

pytestmark = pytest.mark.gpu

# Relative to the largest logit of the compared rows.  float32: rounding of FMA chains
# a few hundred long through a handful of layers, measured at ~1e-6.  bfloat16:
# activations are rounded to 8 bits of mantissa (2^-9 relative) between kernels.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
LENGTHS = {"tiny_a": [70, 96, 45, 33], "tiny_b": [120, 81, 64, 39], "tiny_c": [77, 50, 101, 36],
           "tiny_d": [300, 150, 129, 70], "tiny_e": [257, 140, 66, 200]}
PORTIONS = [7, 2, 13, 3, 2, 5, 2, 31, 2, 4, 16, 2, 9]


def check(got, ref, dtype, what):
    scale = np.abs(ref).max()
    err = np.abs(got.astype(np.float64) - ref).max() / scale
    assert err < TOL[dtype], f"{what}: relative error {err:.3e} (limit {TOL[dtype]:.0e})"
    return err


def cut(n, sizes):
    out, i, k = [], 0, 0
    while i < n:
        s = min(sizes[k % len(sizes)], n - i)
        if n - i - s == 1:  # never leave a single token: portions go down to two, not one
            s += 1
        out.append((i, i + s))
        i += s
        k += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
def test_replay_all_cuttings(name, dtype):
    _replay(name, dtype)


@pytest.mark.parametrize("name,dtype", [("tiny_b", "float32"), ("tiny_d", "bfloat16"), ("tiny_e", "bfloat16")])
def test_replay_all_cuttings_with_cuda_graphs(name, dtype):
    """The same matrix with steps of single tokens replayed from captured graphs, as generation
    runs them: one, two and up to four live requests (graphs of 1, 2 and 4 rows, the last with a
    padding row when three are live)."""
    _replay(name, dtype, ("--cuda-graphs",))


def _replay(name, dtype, flags=()):
    cfg_dict, seed, _ = CONFIGS[name]
    storage = "float32" if dtype == "float32" else "bfloat16"
    mdir = model_dir(name, storage)
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(100 + seed)
    seqs = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in LENGTHS[name]]
    refs = [P.forward(cfg, w, s) for s in seqs]

    # The mixed phase holds up to four requests; size the pool for exactly that, so
    # that the single-request phases before it already reuse pages again and again.
    max_tokens = sum(ceil64(len(s)) for s in seqs)
    extra = {"tiny_a": ("--page-size", "4"), "tiny_e": ("--page-size", "8")}.get(name, ())
    tr = TraceRun(mdir, dtype, max_tokens, tuple(extra) + tuple(flags))
    worst = 0.0
    try:
        # 1. each request alone and whole
        for r, s in enumerate(seqs):
            got = tr.step([(f"w{r}", s, range(len(s)))], end=[f"w{r}"])
            worst = max(worst, check(got, refs[r], dtype, f"{name} whole request {r}"))
        # 2. most of it in one step, the last 32 tokens one by one
        for r, s in enumerate(seqs[:2]):
            n0 = len(s) - 32
            got = tr.step([(f"d{r}", s[:n0], [n0 - 1])])
            check(got, refs[r][n0 - 1:n0], dtype, f"{name} prefix of request {r}")
            for i in range(n0, len(s)):
                got = tr.step([(f"d{r}", [s[i]], [0])], end=[f"d{r}"] if i == len(s) - 1 else [])
                worst = max(worst, check(got, refs[r][i:i + 1], dtype, f"{name} request {r} decoded token {i}"))
        # 3. portions of changing size, down to two tokens
        for r, s in enumerate(seqs):
            spans = cut(len(s), PORTIONS[r:] + PORTIONS[:r])
            for a, b in spans:
                got = tr.step([(f"p{r}", s[a:b], range(b - a))], end=[f"p{r}"] if b == len(s) else [])
                worst = max(worst, check(got, refs[r][a:b], dtype, f"{name} request {r} portion {a}:{b}"))
        # 4. mixed: requests start two steps apart, read their prompt in portions and
        # then go on token by token, beside each other; the earliest ends first and a
        # fifth request (request 0 again) takes over its pages.
        order = [0, 1, 2, 3, 0]
        names = [f"m{k}" for k in range(5)]
        prefill_len = [len(seqs[r]) - 12 for r in order]
        plans = []
        for k, r in enumerate(order):
            spans = cut(prefill_len[k], PORTIONS[k + 3:] + PORTIONS[:k + 3])
            spans += [(i, i + 1) for i in range(prefill_len[k], len(seqs[r]))]
            plans.append(spans)
        start_step = [0, 2, 4, 6, None]
        pos = [0] * 5
        step = 0
        live = set()
        done = set()
        while len(done) < 5:
            for k in range(5):
                if k not in live and k not in done:
                    if start_step[k] is not None and step >= start_step[k]:
                        live.add(k)
                    elif start_step[k] is None and 0 in done:
                        live.add(k)
            entries, ends, expect = [], [], []
            for k in sorted(live):
                a, b = plans[k][pos[k]]
                r = order[k]
                entries.append((names[k], seqs[r][a:b], range(b - a)))
                expect.append(refs[r][a:b])
                pos[k] += 1
                if pos[k] == len(plans[k]):
                    ends.append(names[k])
            assert len(entries) <= 4
            got = tr.step(entries, end=ends)
            worst = max(worst, check(got, np.concatenate(expect), dtype, f"{name} mixed step {step}"))
            for k in list(live):
                if names[k] in ends:
                    live.discard(k)
                    done.add(k)
            step += 1
    finally:
        tr.close()
    print(f"{name} {dtype}: worst relative error {worst:.3e}")

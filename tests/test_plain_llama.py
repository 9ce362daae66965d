"""The plain implementation itself: against the golden outputs of the two upstream
pieces that run on a CPU (sampler mirror, rotary table builder), and against
properties the formulas imply."""

import json
import math
import os

import numpy as np

import plain_llama as P
from tiny_models import TINY_A, TINY_B, model_dir

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_counter_uniform_matches_upstream_mirror():
    g = json.load(open(os.path.join(GOLD, "sampling_golden.json")))
    for seed, key, step, u in g["uniform"]:
        assert P.counter_uniform(seed, key, step) == u
        assert 0.0 <= u < 1.0


def test_temperature_sampling_matches_upstream_flat_and_two_level_walk():
    g = json.load(open(os.path.join(GOLD, "sampling_golden.json")))
    small = np.array(g["small_logits"])
    for t, i, tok in g["small_picks"]:
        assert P.sample_temperature(small, t, P.counter_uniform(5, 2, i)) == tok
    rng = np.random.default_rng(g["big_logits_seed"])
    logits = rng.normal(0.0, 2.0, 128256)
    logits[rng.choice(128256, 20, replace=False)] += 12.0
    for t, i, u, flat, walk in g["big_picks"]:
        assert flat == walk                      # upstream's own claim
        assert P.sample_temperature(logits, t, u) == flat


def test_rope_tables_match_upstream_host_code():
    g = json.load(open(os.path.join(GOLD, "rope_golden.json")))
    scaling = {"factor": g["factor"], "low_freq_factor": g["low_freq_factor"],
               "high_freq_factor": g["high_freq_factor"],
               "original_max_position_embeddings": g["original_max_position_embeddings"]}
    inv32 = P.rope_inv_freq(g["head_dim"], g["theta"], scaling, dtype=np.float32)
    inv64 = P.rope_inv_freq(g["head_dim"], g["theta"], scaling)
    assert np.allclose(inv32, inv64, rtol=1e-6)
    # all three bands of the llama3 rule occur at these constants
    plain = P.rope_inv_freq(g["head_dim"], g["theta"], None)
    ratio = inv64 / plain
    assert np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 1 / g["factor"]) and np.any((ratio > 0.04) & (ratio < 0.99))
    for pos, row in g["rows"].items():
        # One unit in the last place of a float32 inv_freq (powf of libm against numpy's,
        # float32 against float64) moves the angle by pos * inv_freq * 6e-8 <= pos * 6e-8.
        tol = 1e-6 + 3e-7 * int(pos)
        cos32, sin32 = P.rope_tables([int(pos)], inv32, dtype=np.float32)
        assert np.allclose(cos32[0], row["cos"], atol=tol) and np.allclose(sin32[0], row["sin"], atol=tol)
        cos64, sin64 = P.rope_tables([int(pos)], inv64)
        assert np.allclose(cos64[0], row["cos"], atol=tol) and np.allclose(sin64[0], row["sin"], atol=tol)


def test_rope_is_a_rotation_of_pairs_j_and_j_plus_half():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 2, 8))
    inv = P.rope_inv_freq(8, 10000.0)
    cos, sin = P.rope_tables([0, 5, 9], inv)
    y = P.apply_rope(x, cos, sin)
    assert np.allclose(y[0], x[0])                                   # position 0: identity
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))           # norms kept
    a = 5 * inv[1]
    assert np.isclose(y[1, 0, 1], x[1, 0, 1] * math.cos(a) - x[1, 0, 5] * math.sin(a))
    assert np.isclose(y[1, 0, 5], x[1, 0, 1] * math.sin(a) + x[1, 0, 5] * math.cos(a))
    # scores depend on the distance only
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    def score(pq, pk):
        cq, sq = P.rope_tables([pq], inv)
        ck, sk = P.rope_tables([pk], inv)
        return float((P.apply_rope(q, cq, sq) * P.apply_rope(k, ck, sk)).sum())
    assert np.isclose(score(7, 3), score(104, 100))


def test_rms_norm_and_swiglu_formulas():
    x = np.array([[3.0, -4.0, 0.0, 0.0]])
    w = np.array([1.0, 2.0, 1.0, 1.0])
    r = math.sqrt((9 + 16) / 4 + 1e-5)
    assert np.allclose(P.rms_norm(x, w, 1e-5), [[3 / r, -8 / r, 0, 0]])
    wt = {"gate_proj.weight": np.array([[1.0, 0.0]]), "up_proj.weight": np.array([[0.0, 2.0]]),
          "down_proj.weight": np.array([[1.0], [-1.0]])}
    y = P.swiglu_part(np.array([[0.5, 3.0]]), wt, "")
    a = 0.5 / (1 + math.exp(-0.5)) * 6.0
    assert np.allclose(y, [[a, -a]])


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(1)
    T, nq, nkv, d = 9, 4, 2, 8
    q, k, v = rng.normal(size=(T, nq, d)), rng.normal(size=(T, nkv, d)), rng.normal(size=(T, nkv, d))
    out = P.attention(q, k, v)
    assert np.allclose(out[0, 1], v[0, 0]) and np.allclose(out[0, 2], v[0, 1])    # head h reads kv head h // 2
    k2, v2 = k.copy(), v.copy()
    k2[6:], v2[6:] = 7.0, -3.0
    assert np.allclose(P.attention(q, k2, v2)[:6], out[:6])                       # the future is not read
    s = (q[4, 3] @ k[:5, 1].T) / math.sqrt(d)
    p = np.exp(s - s.max())
    assert np.allclose(out[4, 3], (p / p.sum()) @ v[:5, 1])
    w3 = P.attention(q, k, v, window=3)
    s = (q[8, 0] @ k[6:9, 0].T) / math.sqrt(d)
    p = np.exp(s - s.max())
    assert np.allclose(w3[8, 0], (p / p.sum()) @ v[6:9, 0]) and np.allclose(w3[:3], out[:3])


def test_forward_prefix_property_and_tied_head():
    for name, cfg in (("tiny_a", TINY_A), ("tiny_b", TINY_B)):
        c, w = P.read_model_dir(model_dir(name))
        toks = list(np.random.default_rng(3).integers(0, cfg["vocab_size"], 12))
        full = P.forward(c, w, toks)
        assert full.shape == (12, cfg["vocab_size"]) and np.isfinite(full).all()
        assert np.allclose(P.forward(c, w, toks[:7]), full[:7], atol=1e-12)
        assert ("lm_head.weight" in w) == (not cfg["tie_word_embeddings"])


def test_sampling_rules():
    l = np.array([1.0, 3.0, 3.0, -2.0])
    assert P.argmax_lowest(l) == 1                                    # the lower index wins a tie
    assert P.sample(l, 0.0, 0, 0, 0) == 1
    pen = P.penalise(l, [1, 3], 1.15)
    assert np.allclose(pen, [1.0, 3.0 / 1.15, 3.0, -2.0 * 1.15]) and P.argmax_lowest(pen) == 2
    assert P.sample_temperature(l, 1.0, 0.0) == 0 and P.sample_temperature(l, 1.0, 1 - 2 ** -24) == 3
    assert P.round_bf16(np.array([1.00390625]))[0] == 1.0 and P.round_bf16(np.array([1.01171875]))[0] == 1.015625

"""Plain, slow restatement of the Llama dense decoder, sampling included.

Whole sequences, no cache, numpy only, one function per part.  It shares no code
with the package under test: it even reads ``model.safetensors`` with its own
few lines.  Every function cites the lines of the upstream project
(thientd05/kv_cache_optimization_for_llm, paths relative to its root) whose
formula it restates.

The upstream model code cannot run without a GPU (every op is a CUDA kernel or a
cuBLAS call and every size is a compile-time constant), so the model formulas
here were written from reading those lines.  Three things of upstream anchor this
file through ``tests/golden/``: its numpy sampler mirror
(``python/sampling_reference.py``) and the host half of ``initRopeFrequencies``,
which run on a CPU, and the tokens that its unmodified engine, compiled for a
B200, generated on a Llama-3.2-1B-shaped model with random weights
(``tests/golden/upstream_tokens_llama1b.json``): ``tests/test_upstream_golden_gpu.py``
checks that those tokens are the best under the logits of this file and of the
engine.

Arithmetic is float64 unless a function takes ``dtype``; the engine's float32
path must agree with it to float32 rounding, the bfloat16 path to bfloat16
rounding.
"""

from __future__ import annotations

import json
import math
import struct

import numpy as np


# --------------------------------------------------------------------------- files

_ST_DTYPES = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "F16": np.float16}


def read_safetensors(path):
    """u64 header length, JSON header, raw payload (base/src/model.cu:33-64)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        payload = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = payload[lo:hi]
        if meta["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u16.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = arr.reshape(meta["shape"]).astype(np.float64)
    return out


def read_model_dir(model_dir):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors")


def round_bf16(x):
    """Round-to-nearest-even to bfloat16, returned as float64."""
    a = np.asarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64)


# --------------------------------------------------------------------------- parts

def rope_inv_freq(head_dim, theta, scaling=None, dtype=np.float64):
    """inv_freq_i = 1/theta^(2i/d), then the llama3 three-band rescale
    (base/src/kernels.cu:58-83).  ``scaling`` is config.json's ``rope_scaling``
    dict or None; ``dtype=np.float32`` repeats upstream's single precision."""
    f = dtype
    half = head_dim // 2
    i = np.arange(half, dtype=f)
    inv = (f(1.0) / np.power(f(theta), (f(2.0) * i) / f(head_dim))).astype(f)
    if not scaling:
        return inv
    factor = f(scaling["factor"])
    low_ff = f(scaling["low_freq_factor"])
    high_ff = f(scaling["high_freq_factor"])
    orig = f(scaling["original_max_position_embeddings"])
    low_w = orig / low_ff
    high_w = orig / high_ff
    out = inv.copy()
    for k in range(half):
        wavelen = f(2.0) * f(math.pi) / inv[k]
        if wavelen > low_w:
            out[k] = inv[k] / factor
        elif wavelen >= high_w:
            smooth = (orig / wavelen - low_ff) / (high_ff - low_ff)
            out[k] = (f(1.0) - smooth) * (inv[k] / factor) + smooth * inv[k]
    return out


def rope_tables(positions, inv_freq, dtype=np.float64):
    """angle = pos * inv_freq_i; cos and sin per (pos, i) (base/src/kernels.cu:88-99)."""
    ang = np.asarray(positions, dtype=dtype)[:, None] * inv_freq.astype(dtype)[None, :]
    return np.cos(ang), np.sin(ang)


def apply_rope(x, cos, sin):
    """Rotate-half on [T, heads, d]: pairs (j, j+d/2):
    x[j] = x1*c - x2*s ; x[j+d/2] = x1*s + x2*c (base/src/kernels.cu:289-319)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1)


def rms_norm(x, w, eps):
    """y = (x / sqrt(mean(x^2) + eps)) * w, divide first, plain weight
    (base/src/kernels.cu:10-36)."""
    r = np.sqrt((x * x).sum(-1, keepdims=True) / x.shape[-1] + eps)
    return (x / r) * w


def linear(x, w):
    """y = x . W^T with W [out, in], no bias (base/src/engine.cu:643-671)."""
    return x @ w.T


def attention(q, k, v, window=None):
    """Causal grouped-query attention on one sequence, [T, heads, d] each.
    kv head = q head // (nq/nkv) (base/src/kernels.cu:372); score = (q.k)/sqrt(d),
    keys j <= i (:387,:422,:431); softmax; weighted sum of v (:436-464).
    ``window`` keeps only the newest ``window`` keys (j > i - window); upstream
    has no window, None is its behaviour."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = np.zeros_like(q)
    for h in range(nq):
        hk = h // group
        s = (q[:, h, :] @ k[:, hk, :].T) / math.sqrt(d)
        i = np.arange(T)[:, None]
        j = np.arange(T)[None, :]
        mask = j <= i
        if window is not None:
            mask &= j > i - window
        s = np.where(mask, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(-1, keepdims=True)
        out[:, h, :] = p @ v[:, hk, :]
    return out


def gqa_attention_part(x, w, prefix, cfg, positions, inv_freq, window=None):
    """q,k,v from the same normed input, RoPE on q and k (not v), attention,
    output projection (base/src/engine.cu:653-762)."""
    T = x.shape[0]
    nq = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nq)
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    q = linear(x, w[prefix + "q_proj.weight"]).reshape(T, nq, d)
    k = linear(x, w[prefix + "k_proj.weight"]).reshape(T, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"]).reshape(T, nkv, d)
    cos, sin = rope_tables(positions, inv_freq)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    a = attention(q, k, v, window=window).reshape(T, nq * d)
    return linear(a, w[prefix + "o_proj.weight"])


def swiglu_part(x, w, prefix):
    """a = g * (1/(1+exp(-g))) * u ; y = a . W_down^T
    (base/src/kernels.cu:45-52, base/src/engine.cu:780-855)."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    a = g * (1.0 / (1.0 + np.exp(-g))) * u
    return linear(a, w[prefix + "down_proj.weight"])


def decoder_layer(h, w, layer, cfg, positions, inv_freq):
    """h += Attn(RMSNorm_in(h)); h += MLP(RMSNorm_post(h)) (base/src/engine.cu:639-859)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    h = h + gqa_attention_part(x, w, p + "self_attn.", cfg, positions, inv_freq)
    x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    h = h + swiglu_part(x, w, p + "mlp.")
    return h


def forward(cfg, w, tokens, rows=None):
    """Logits [T, vocab] of one whole sequence: embedding gather (no scale),
    the layers, final norm, LM head = embedding when tied
    (base/src/engine.cu:637,639-890).  ``rows``: the positions whose logits are
    wanted (the head then runs on those rows only, as upstream's does on the last
    row of each prompt, base/src/engine.cu:862-890); None: all."""
    tokens = np.asarray(tokens, dtype=np.int64)
    nq = cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    inv_freq = rope_inv_freq(d, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    positions = np.arange(len(tokens))
    h = w["model.embed_tokens.weight"][tokens]
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, layer, cfg, positions, inv_freq)
    if rows is not None:
        h = h[np.asarray(list(rows), dtype=np.int64)]
    x = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------------- sampling

_M64 = (1 << 64) - 1


def counter_uniform(seed, seq_key, step):
    """splitmix64 finaliser of (key<<32 ^ step) mixed with the seed, top 24 bits
    (base/src/kernels.cu:638-649)."""
    z = ((seq_key << 32) ^ step) & _M64
    z ^= (seed * 0x9E3779B97F4A7C15) & _M64
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z = z ^ (z >> 31)
    return (z >> 40) * (1.0 / 16777216.0)


def penalise(logits, seen, penalty):
    """Seen tokens: positive logit divided by the penalty, negative multiplied
    (base/src/kernels.cu:504-513)."""
    out = np.array(logits, dtype=np.float64)
    if penalty != 1.0:
        for t in set(seen):
            out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out


def argmax_lowest(logits):
    """Greedy pick; the lower index wins a tie (base/src/kernels.cu:489-496)."""
    return int(np.argmax(logits))


def sample_temperature(logits, temperature, u):
    """p ~ exp((l - max)/T); token = first index whose inclusive prefix sum
    exceeds u*total (base/src/kernels.cu:676-835, python/sampling_reference.py:85-89)."""
    w = np.exp((logits - logits.max()) / temperature)
    cdf = np.cumsum(w)
    return int(min(np.searchsorted(cdf, u * cdf[-1], side="right"), len(logits) - 1))


def sample(logits, temperature, seed, key, pos, seen=(), penalty=1.0):
    """temperature <= 0 is greedy (base/src/engine.cu:132-158).  ``pos`` is the
    index the sampled token will have in its sequence."""
    l = penalise(logits, seen, penalty)
    if temperature <= 0:
        return argmax_lowest(l)
    return sample_temperature(l, temperature, counter_uniform(seed, key, pos))


def generate(cfg, w, prompt, max_tokens, temperature=0.0, seed=0, key=0, penalty=1.0, eos=()):
    """Token-by-token generation by full recompute; returns the new tokens.
    A sampled stop token ends the sequence and is not returned
    (base/src/engine.cu:919-977,1275-1308)."""
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(cfg, w, seq)[-1]
        tok = sample(logits, temperature, seed, key, len(seq), seen=out, penalty=penalty)
        if tok in eos:
            break
        out.append(tok)
        seq.append(tok)
    return out

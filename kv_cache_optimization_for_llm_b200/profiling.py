"""Small workloads for profilers: a few decode steps or one prompt portion of a
random-weights model, with the CUDA profiler range switched on around them only.

    python -m kv_cache_optimization_for_llm_b200.profiling decode  --batch 8 --layers 4 --steps 2
    python -m kv_cache_optimization_for_llm_b200.profiling prefill --tokens 2048 --layers 4
    python -m kv_cache_optimization_for_llm_b200.profiling attention --batch 8 --context 16000
    python -m kv_cache_optimization_for_llm_b200.profiling timeline --batch 8 --layers 16

``timeline`` prints, for the kernels of one captured decode step, the medians over their blocks
of the phase stamps that the product kernel and the decode attention kernel write themselves
(globaltimer), relative to the moment the kernel in front of each had finished.

``attention`` times the decode attention kernel alone (CUDA events around a graph of 16
launches over 16 layers' caches, so that the keys and values do not come from L2) and prints
microseconds per launch and the bandwidth over the keys and values it has to read.

Under ``ncu --profile-from-start off`` only the bracketed work is captured.  Fewer
layers than the full model keep a capture short and its memory small; the kernels and
their sizes per layer are those of the full model.  The default shape is Llama-3.2-1B
(the sizes of its config.json); ``--shape 3b`` and ``--shape 8b`` are Llama-3.2-3B and
Llama-3.1-8B, ``--config-json`` takes any other config.json.
"""

from __future__ import annotations

import argparse
import json
import sys
import time

LLAMA_3_2_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
}
_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
# The sizes of the config.json files of three Llama models (random weights are made for them).
SHAPES = {
    "1b": LLAMA_3_2_1B,
    "3b": dict(LLAMA_3_2_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8,
               head_dim=128, intermediate_size=8192, rope_scaling=dict(_ROPE, factor=32.0)),
    "8b": dict(LLAMA_3_2_1B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=14336, tie_word_embeddings=False, rope_scaling=dict(_ROPE, factor=8.0)),
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["decode", "prefill", "attention", "timeline"])
    ap.add_argument("--config-json", help="a config.json; default: the Llama-3.2-1B shape")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1b",
                    help="the sizes of Llama-3.2-1B, Llama-3.2-3B or Llama-3.1-8B (without --config-json)")
    ap.add_argument("--layers", type=int, default=None, help="override num_hidden_layers")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512, help="prompt length of the decode requests")
    ap.add_argument("--steps", type=int, default=2, help="decode steps inside the profiler range")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the prefill step")
    ap.add_argument("--context", type=int, default=640, help="context length of every request (attention)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--spread", action="store_true",
                    help="timeline: also the 10th and 90th percentile and the extremes over the blocks of each phase")
    a = ap.parse_args(argv)

    import numpy as np
    import torch

    from . import LLM, SamplingParams
    from .engine.batch import StepEntry

    cfg = json.load(open(a.config_json)) if a.config_json else dict(SHAPES[a.shape])
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    if a.what == "attention":
        return _attention_alone(cfg, a.batch, a.context)
    if a.what == "timeline":
        return _timeline(cfg, a.batch, a.prompt, a.spread)
    page = 16
    need = a.batch * (a.prompt + 64 + a.steps) if a.what == "decode" else a.tokens
    llm = LLM.from_random(cfg, dtype=a.dtype, page_size=page, num_pages=need // page + 64,
                          max_num_seqs=max(a.batch, 1), max_num_batched_tokens=max(2048, a.tokens),
                          max_model_len=4096, use_cuda_graphs=not a.no_graphs)
    eng = llm.engine
    rng = np.random.default_rng(0)
    vocab = eng.runner.vocab_size
    prof = torch.cuda.cudart()
    if a.what == "prefill":
        toks = rng.integers(0, vocab, a.tokens).tolist()
        for k in range(2):                                   # warm-up
            eng.runner.step([StepEntry(100 + k, toks, 0, [a.tokens - 1])])
            eng.runner.release(100 + k)
        torch.cuda.synchronize()
        prof.cudaProfilerStart()
        t0 = time.perf_counter()
        eng.runner.step([StepEntry(200, toks, 0, [a.tokens - 1])])
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        prof.cudaProfilerStop()
        print(f"prefill of {a.tokens} tokens, {cfg['num_hidden_layers']} layers: {ms:.3f} ms")
        return 0
    sp = SamplingParams(max_tokens=48 + a.steps, ignore_eos=True)
    ids = [eng.add_request(rng.integers(0, vocab, a.prompt).tolist(), sp) for _ in range(a.batch)]
    produced = {i: 0 for i in ids}
    while min(produced.values()) < 1:
        for ev in eng.step():
            if ev.token is not None:
                produced[ev.request_id] += 1
    for _ in range(4):                                       # warm-up, graph capture
        eng.step()
    torch.cuda.synchronize()
    prof.cudaProfilerStart()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        eng.step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / a.steps
    prof.cudaProfilerStop()
    print(f"decode, batch {a.batch}, {cfg['num_hidden_layers']} layers: {ms:.3f} ms per step")
    return 0


def _timeline(cfg, batch: int, prompt: int, spread: bool = False) -> int:
    """Phase stamps of the product and attention kernels inside a captured decode step."""
    import numpy as np
    import torch

    from . import LLM, SamplingParams, ops
    pool = [torch.zeros(4096, 8, dtype=torch.int64, device="cuda") for _ in range(8 * cfg["num_hidden_layers"] + 8)]
    calls = []          # (kind, trace buffer) in launch order

    def buffer_for(kind):
        t = pool[len(calls) % len(pool)]
        calls.append((kind, t))
        return t
    names = {}
    plain, fused, attn = ops.gemm_skinny, ops.gemm_skinny_fused, ops.decode_attention_mma

    def kind_of(w, extra=""):
        return names.setdefault((w.shape[0], w.shape[1], extra), f"product {w.shape[0]}x{w.shape[1]}{extra}")
    ops.gemm_skinny = lambda x, w, dt, st, x_is_static=False, trace=None, **kw: plain(
        x, w, dt, st, x_is_static, buffer_for(kind_of(w)), **kw)
    ops.gemm_skinny_fused = lambda x, w, st, **kw: fused(
        x, w, st, **{**kw, "trace": buffer_for(kind_of(w, " +residual" if kw.get("into") is not None else
                                                         (" +silu" if kw.get("epilogue") == "swiglu" else "")))})
    ops.decode_attention_mma = lambda *args, **kw: attn(*args, **{**kw, "trace": buffer_for("decode attention")})

    llm = LLM.from_random(cfg, dtype="bfloat16", page_size=16, num_pages=batch * (prompt + 128) // 16 + 64,
                          max_num_seqs=batch, max_num_batched_tokens=2048, max_model_len=4096)
    eng = llm.engine
    rng = np.random.default_rng(0)
    sp = SamplingParams(max_tokens=64, ignore_eos=True)
    ids = [eng.add_request(rng.integers(0, eng.runner.vocab_size, prompt).tolist(), sp) for _ in range(batch)]
    produced = {i: 0 for i in ids}
    while min(produced.values()) < 1:
        for ev in eng.step():
            if ev.token is not None:
                produced[ev.request_id] += 1
    for _ in range(4):
        eng.step()
    torch.cuda.synchronize()
    # the graph was captured by the last forward pass that went through the hooks: its calls are the tail of the list
    n = 5 * cfg["num_hidden_layers"] + 1
    captured = calls[-n:]
    for t in pool:
        t.zero_()
    for _ in range(4):
        eng.step()
    torch.cuda.synchronize()
    gemm_cols = [("first tile", 3), ("last product issued", 4), ("accumulator complete", 5), ("partials here", 7), ("stored", 6)]
    attn_cols = [("queries ready", 2), ("first class walked", 3), ("partials sent", 4), ("cluster met", 5), ("stored", 6)]
    rows, t_first, spreads = {}, None, {}
    for kind, t in captured:
        a = t.cpu().numpy().astype(np.float64)
        a = a[a[:, 0] > 0]
        if len(a) == 0:
            continue
        is_attn = kind == "decode attention"
        dep = np.median(a[:, 1 if is_attn else 2])
        if t_first is None:
            t_first = a[:, 0].min()
        vals = [(np.median(a[:, 0]) - dep) / 1e3]
        for _, col in (attn_cols if is_attn else gemm_cols):
            c = a[:, col]
            c = c[c > 0]
            vals.append((np.median(c) - dep) / 1e3 if len(c) else float("nan"))
        vals.append((a[:, 6].max() - dep) / 1e3)
        rows.setdefault(kind, []).append(vals)
        if spread:
            pcs = []
            for _, col in [("blocks start", 0)] + (attn_cols if is_attn else gemm_cols):
                c = a[:, col]
                c = c[c > 0]
                pcs.append([(f(c) - dep) / 1e3 if len(c) else float("nan") for f in
                            (np.min, lambda x: np.percentile(x, 10), np.median, lambda x: np.percentile(x, 90), np.max)])
            spreads.setdefault(kind, []).append(pcs)
        t_last = a[:, 6].max()
    print(f"decode step, batch {batch}: {(t_last - t_first) / 1e3:.1f} us from the first product's first block to the LM head's last store")
    print("microseconds relative to the end of each kernel's wait for the kernel in front (medians over blocks, mean over layers)")
    for kind, v in rows.items():
        arr = np.array(v)
        m = np.array([np.nanmean(c) if np.isfinite(c).any() else float("nan") for c in arr.T])
        cols = attn_cols if kind == "decode attention" else gemm_cols
        txt = "  ".join(f"{nm} {x:5.1f}" for (nm, _), x in zip(cols, m[1:-1]))
        print(f"  {kind:32s} x{len(v):3d}  blocks start {m[0]:6.1f}  {txt}  last block done {m[-1]:5.1f}")
        if spread:
            sp_mean = np.nanmean(np.array(spreads[kind]), axis=0)      # [phase, 5]
            for (nm, _), q in zip([("blocks start", 0)] + cols, sp_mean):
                print(f"      {nm:22s} min {q[0]:6.1f}  p10 {q[1]:6.1f}  median {q[2]:6.1f}  p90 {q[3]:6.1f}  max {q[4]:6.1f}")
    return 0


def _attention_alone(cfg, batch: int, context: int) -> int:
    import math

    import torch

    from . import ops
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    page, layers = 16, 16
    pages_per = -(-context // page)
    n_pages = batch * pages_per
    kv = torch.randn(layers, 2, n_pages + 1, nkv, page, d, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").view(batch, pages_per).contiguous()
    qkv = torch.randn(batch, (nq + 2 * nkv) * d, device="cuda", dtype=torch.bfloat16)
    q_start = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    ctx_len = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cos = torch.ones(context, d // 2, device="cuda")
    sin = torch.zeros(context, d // 2, device="cuda")

    def run():
        for layer in range(layers):
            ops.decode_attention_mma(qkv, kv[layer, 0], kv[layer, 1], True, table, q_start, ctx_len, cos, sin, d, nq, nkv,
                                     d, 1 / math.sqrt(d), None, status, max_ctx=context)
    run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(3):
        graph.replay()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(20):
        graph.replay()
    t1.record()
    torch.cuda.synchronize()
    us = t0.elapsed_time(t1) * 1000 / 20 / layers
    nbytes = batch * context * nkv * d * 2 * 2
    print(f"decode attention, batch {batch}, context {context}: {us:.1f} us per launch, "
          f"{nbytes / us / 1e3:.0f} GB/s over {nbytes / 1e6:.0f} MB of keys and values")
    return 0


if __name__ == "__main__":
    sys.exit(main())

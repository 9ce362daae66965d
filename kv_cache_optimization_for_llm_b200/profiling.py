"""Small workloads for profilers: a few decode steps or one prompt portion of a
random-weights model, with the CUDA profiler range switched on around them only.

    python -m kv_cache_optimization_for_llm_b200.profiling decode  --batch 8 --layers 4 --steps 2
    python -m kv_cache_optimization_for_llm_b200.profiling prefill --tokens 2048 --layers 4
    python -m kv_cache_optimization_for_llm_b200.profiling attention --batch 8 --context 16000

``attention`` times the decode attention kernel alone (CUDA events around a graph of 16
launches over 16 layers' caches, so that the keys and values do not come from L2) and prints
microseconds per launch and the bandwidth over the keys and values it has to read.

Under ``ncu --profile-from-start off`` only the bracketed work is captured.  Fewer
layers than the full model keep a capture short and its memory small; the kernels and
their sizes per layer are those of the full model.  The default shape is Llama-3.2-1B
(the sizes of its config.json); ``--config-json`` takes any other config.json.
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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["decode", "prefill", "attention"])
    ap.add_argument("--config-json", help="a config.json; default: the Llama-3.2-1B shape")
    ap.add_argument("--layers", type=int, default=None, help="override num_hidden_layers")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512, help="prompt length of the decode requests")
    ap.add_argument("--steps", type=int, default=2, help="decode steps inside the profiler range")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the prefill step")
    ap.add_argument("--context", type=int, default=640, help="context length of every request (attention)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--no-graphs", action="store_true")
    a = ap.parse_args(argv)

    import numpy as np
    import torch

    from . import LLM, SamplingParams
    from .engine.batch import StepEntry

    cfg = json.load(open(a.config_json)) if a.config_json else dict(LLAMA_3_2_1B)
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    if a.what == "attention":
        return _attention_alone(cfg, a.batch, a.context)
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

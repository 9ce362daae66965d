#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Llama-3.2-1B size, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A "step" is one decode step of ``--batch`` requests.  Each request is a 512-token
uniform-random prompt; after the prompts are read, W decode steps warm up and
exactly K are timed, once on the device (CUDA events on the launching stream:
``value``) and once end to end through the Python entry point (host token ids in,
sampled ids out at every step: ``e2e``).  Weights are random (N(0, 0.02), norms
1 + N(0, 0.02)), bfloat16, 16-token pages, context limit 4096.  One JSON line goes
to standard output; progress goes to standard error.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
}
_LLAMA3_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                "original_max_position_embeddings": 8192}
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8,
                head_dim=128, intermediate_size=8192, rope_scaling=dict(_LLAMA3_ROPE, factor=32.0))
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(_LLAMA3_ROPE, factor=8.0))
# The two serving workloads beside the headline: continuous batching under Poisson arrivals at the
# 3B shape, and 64 long requests at the 8B shape in a pool that cannot hold them all.
WORKLOADS = {
    "serve3b": {"model": LLAMA_3B, "name": "Llama-3.2-3B shape", "requests": 256, "prompt_len": (128, 2048),
                "output_len": (64, 512), "arrival_rate": 64.0, "context_len": 8192, "max_num_seqs": 256,
                "pool_fraction_of_need": 0.6},
    "stress8b": {"model": LLAMA_8B, "name": "Llama-3.1-8B shape", "requests": 64, "prompt_len": (4096, 4096),
                 "output_len": (512, 512), "arrival_rate": 0.0, "context_len": 16384, "max_num_seqs": 64,
                 "pool_fraction_of_need": 0.75},
}
FULL_LAYERS = LLAMA_1B["num_hidden_layers"]
CONTEXT_LEN = 4096
PROMPT_LEN = 512
NEW_TOKENS = 256
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def log(msg):
    print(f"[bench] {msg}", file=sys.stderr, flush=True)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except Exception as e:  # an unreadable file must not cost the run
            log(f"MEASURED_PEAKS.json could not be used ({e}); falling back")
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, windows):
        """Clocks of the samples that fall inside the timed windows [(t0, t1), ...]."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [(t, line) for t, line in self.lines if any(a <= t <= b for a, b in windows)]
        if len(inside) < 3:
            # timed regions shorter than the sampling period: take the samples next to them as well
            inside = [(t, line) for t, line in self.lines if any(a - 0.25 <= t <= b + 0.25 for a, b in windows)]
        for t, line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def model_numbers(cfg, layers):
    """Bytes and FLOPs of this model's steps, from the configuration."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    layer_matrix = (nq * d + 2 * nkv * d) * H + H * nq * d + 3 * I * H
    weight_elems = layers * (layer_matrix + 2 * H) + V * H + H
    return {
        "weight_bytes": 2 * weight_elems,                   # bfloat16, every weight read once per step
        "kv_bytes_per_token": layers * 2 * nkv * d * 2,      # keys and values, bfloat16
        "layer_matrix_elems": layer_matrix,
        "attn_flops_per_pair": 4 * nq * d,                   # q.k and p.v per (query, key) pair, all heads
    }


def prefill_flops(cfg, layers, T):
    n = model_numbers(cfg, layers)
    gemm = 2 * T * layers * n["layer_matrix_elems"] + 2 * cfg["vocab_size"] * cfg["hidden_size"]
    attn = layers * n["attn_flops_per_pair"] * T * (T + 1) // 2
    return gemm + attn


def run_decode(llm, batch, steps, warmup, end_to_end, seed):
    """Reads ``batch`` prompts, warms up, times ``steps`` decode steps.  Returns
    (seconds, mean context during the timed steps, launches, (t0, t1) wall window)."""
    import numpy as np
    import torch
    from kv_cache_optimization_for_llm_b200 import SamplingParams, ops
    eng = llm.engine
    rng = np.random.default_rng(seed)
    vocab = eng.runner.vocab_size
    sp = SamplingParams(max_tokens=NEW_TOKENS, ignore_eos=True)
    ids = [eng.add_request(rng.integers(0, vocab, PROMPT_LEN).tolist(), sp) for _ in range(batch)]
    produced = {i: 0 for i in ids}
    while min(produced.values()) < 1:          # read the prompts (mixed steps until every request decodes)
        for ev in eng.step():
            if ev.token is not None:
                produced[ev.request_id] += 1
    lead = max(produced.values())
    # Warm-up: steps of single tokens only (the timed kind), at least three even when some
    # requests already decoded while others still read their prompts.
    for _ in range(max(3, warmup - (lead - 1))):
        eng.step()
        lead += 1
    if lead + steps > NEW_TOKENS:
        raise SystemExit(f"{lead} tokens were produced before timing; {steps} more exceed the budget of {NEW_TOKENS}")
    torch.cuda.synchronize()
    ctx0 = PROMPT_LEN + max(len(eng.output(i)) for i in ids)
    launches0 = ops.launch_count + eng.runner.graph_launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    start.record()
    n_tok = 0
    for _ in range(steps):
        n_tok += sum(1 for ev in eng.step() if ev.token is not None)
    stop.record()
    torch.cuda.synchronize()
    w1 = time.perf_counter()
    assert n_tok == batch * steps, f"{n_tok} tokens from {batch} requests in {steps} steps"
    launches = ops.launch_count + eng.runner.graph_launches - launches0
    seconds = (w1 - w0) if end_to_end else start.elapsed_time(stop) / 1000.0
    run_decode.h2d_bytes = eng.runner.builder.last_h2d_bytes      # of one decode step of this batch
    for i in ids:
        eng.abort(i)
    assert eng.runner.manager.check() == "" and eng.runner.manager.live_requests() == 0
    return seconds, ctx0 + (steps - 1) / 2.0, launches, (w0, w1)


def run_prefill(llm, reps, warmup, seed):
    import numpy as np
    import torch
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    r = llm.engine.runner
    rng = np.random.default_rng(seed)
    toks = rng.integers(0, r.vocab_size, PREFILL_TOKENS).tolist()
    times = []
    for k in range(warmup + reps):
        rid = 10_000_000 + k
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        logits = r.step([StepEntry(rid, toks, 0, [PREFILL_TOKENS - 1])])
        stop.record()
        torch.cuda.synchronize()
        assert logits.shape == (1, r.vocab_size)
        r.release(rid)
        if k >= warmup:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def run_first_token(llm, prompt_len, reps, warmup, seed):
    """Milliseconds from handing one prompt of ``prompt_len`` tokens to an idle engine to its first
    token on the host, through add_request and step (median)."""
    import numpy as np
    import torch
    from kv_cache_optimization_for_llm_b200 import SamplingParams
    eng = llm.engine
    rng = np.random.default_rng(seed)
    times = []
    for k in range(warmup + reps):
        prompt = rng.integers(0, eng.runner.vocab_size, prompt_len).tolist()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        rid = eng.add_request(prompt, SamplingParams(max_tokens=2, ignore_eos=True))
        first = None
        while first is None:
            for ev in eng.step():
                if ev.request_id == rid and ev.token is not None and first is None:
                    first = time.perf_counter()
        while eng.has_unfinished():
            eng.step()
        if k >= warmup:
            times.append((first - t0) * 1e3)
    return statistics.median(times)


def run_value_check(cfg, layers=2):
    """The numbers behind the timings: a model of the benchmark's widths with ``layers`` layers is written to a
    temporary folder and its logits, on the paths that the benchmark times (one 2048-token portion; eight
    requests decoding beside each other from 512-token prompts, replayed from a captured graph), are compared
    with the plain implementation under tests/ at the limit the tests use for bfloat16."""
    import shutil
    import tempfile

    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama as P
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    from kv_cache_optimization_for_llm_b200.weights import write_random_model

    limit = 4e-2
    small = dict(cfg)
    small["num_hidden_layers"] = layers
    d = tempfile.mkdtemp(prefix="kvb200_bench_check_")
    try:
        write_random_model(d, small, seed=0, std=0.02, storage_dtype="bfloat16")
        pcfg, w = P.read_model_dir(d)
        r = ModelRunner(d, EngineConfig(dtype="bfloat16", page_size=PAGE_SIZE, num_pages=8 * 40 + 140, max_num_seqs=8,
                                        max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT_LEN))
        rng = np.random.default_rng(5)
        worst = {}

        def err(got, ref):
            return float(np.abs(got.astype(np.float64) - ref).max() / np.abs(ref).max())

        seq = rng.integers(0, cfg["vocab_size"], PREFILL_TOKENS).tolist()
        rows = [0, 777, PREFILL_TOKENS - 1]
        got = r.step([StepEntry(999, seq, 0, rows)]).float().cpu().numpy()
        r.release(999)
        worst["prefill_2048"] = err(got, P.forward(pcfg, w, seq, rows=rows))
        seqs = [rng.integers(0, cfg["vocab_size"], PROMPT_LEN + 3).tolist() for _ in range(8)]
        r.step([StepEntry(i, s_[:PROMPT_LEN], 0, []) for i, s_ in enumerate(seqs)][:4])
        r.step([StepEntry(i, s_[:PROMPT_LEN], 0, []) for i, s_ in enumerate(seqs)][4:])
        got = None
        for t in range(PROMPT_LEN, PROMPT_LEN + 3):
            got = r.step([StepEntry(i, [s_[t]], t, [0]) for i, s_ in enumerate(seqs)]).float().cpu().numpy()
        ref = np.stack([P.forward(pcfg, w, s_, rows=[PROMPT_LEN + 2])[0] for s_ in seqs])
        worst["decode_b8"] = err(got, ref)
        kinds = dict(r.step_kinds)
    finally:
        shutil.rmtree(d, ignore_errors=True)
    ok = all(v < limit for v in worst.values())
    return {"ok": ok, "limit": limit, "layers": layers, "worst_relative_error": {k: round(v, 5) for k, v in worst.items()},
            "step_kinds": kinds}


def _pct(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(p / 100.0 * (len(xs) - 1))))] if xs else None


def run_workload(name, seed=0):
    """One of WORKLOADS through the engine's own entry points (add_request, step), requests arriving
    in real time.  Every request must emit exactly its budget and no page may be lost; returns
    output tokens a second, time to the first token and time per further token, and what the
    scheduler had to drop and recompute."""
    import gc
    import numpy as np
    import torch
    from kv_cache_optimization_for_llm_b200 import LLM, SamplingParams
    wl = WORKLOADS[name]
    cfg = dict(wl["model"])
    rng = np.random.default_rng(seed)
    n = wl["requests"]
    p_len = rng.integers(wl["prompt_len"][0], wl["prompt_len"][1] + 1, n)
    o_len = rng.integers(wl["output_len"][0], wl["output_len"][1] + 1, n)
    gaps = rng.exponential(1.0 / wl["arrival_rate"], n) if wl["arrival_rate"] > 0 else np.zeros(n)
    arrive = np.cumsum(gaps) - gaps[0]
    need_tokens = int((p_len + o_len).sum())
    pool_tokens = int(need_tokens * wl["pool_fraction_of_need"])
    num_pages = max(pool_tokens // PAGE_SIZE, (int((p_len + o_len).max()) + PAGE_SIZE) // PAGE_SIZE + 1)
    log(f"{name}: building {wl['name']}, {cfg['num_hidden_layers']} layers, pool of {num_pages} pages "
        f"({num_pages * PAGE_SIZE} tokens; all requests together need {need_tokens})")
    llm = LLM.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=num_pages,
                          max_num_seqs=wl["max_num_seqs"], max_num_batched_tokens=PREFILL_TOKENS,
                          max_model_len=wl["context_len"], capture_graphs_at_start=True)
    eng = llm.engine
    kv_bytes = eng.runner.cache.bytes_per_page() * num_pages
    prompts = [rng.integers(0, cfg["vocab_size"], int(k)).tolist() for k in p_len]
    # warm-up: a prompt of two portions and a few decode steps (kernels loaded, allocator warm)
    eng.generate([prompts[0][:128] * 20], SamplingParams(max_tokens=4, ignore_eos=True))
    torch.cuda.synchronize()
    first, last, count = {}, {}, {i: 0 for i in range(n)}
    errors = []
    nxt = 0
    t0 = time.perf_counter()
    while nxt < n or eng.has_unfinished():
        now = time.perf_counter() - t0
        while nxt < n and arrive[nxt] <= now:
            eng.add_request(prompts[nxt], SamplingParams(max_tokens=int(o_len[nxt]), ignore_eos=True), request_id=1000 + nxt)
            nxt += 1
        if not eng.has_unfinished():
            time.sleep(max(0.0, min(0.001, arrive[nxt] - now)))
            continue
        for ev in eng.step():
            t = time.perf_counter() - t0
            i = ev.request_id - 1000
            if ev.token is not None:
                count[i] += 1
                first.setdefault(i, t)
                last[i] = t
            if ev.finished and ev.reason != "length":
                errors.append((i, ev.reason))
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    st = eng.stats()
    wrong = [i for i in range(n) if count[i] != int(o_len[i])]
    assert not errors and not wrong, f"{name}: requests ended early {errors[:3]} or with other counts than their budget {wrong[:3]}"
    assert eng.runner.manager.check() == "" and st["free_pages"] == [num_pages], "a page was lost"
    ttft = [1000.0 * (first[i] - arrive[i]) for i in range(n)]
    tpot = [1000.0 * (last[i] - first[i]) / (count[i] - 1) for i in range(n) if count[i] > 1]
    out_tokens = int(o_len.sum())
    res = {
        "value": round(out_tokens / seconds, 1), "unit": "output tokens/s", "seconds": round(seconds, 3),
        "requests": n, "prompt_tokens": int(p_len.sum()), "output_tokens": out_tokens,
        "total_tokens_per_s": round((out_tokens + int(p_len.sum())) / seconds, 1),
        "ttft_ms": {"p50": round(_pct(ttft, 50), 2), "p99": round(_pct(ttft, 99), 2)},
        "per_token_ms": {"p50": round(_pct(tpot, 50), 3), "p99": round(_pct(tpot, 99), 3)},
        "steps": int(st["steps"]), "preemptions": int(st["preemptions"]), "recomputed_tokens": int(st["recomputed_tokens"]),
        "step_kinds": st.get("step_kinds"),
        "config": {"model": wl["name"], "layers": cfg["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
                   "heads": f"{cfg['num_attention_heads']}/{cfg['num_key_value_heads']}", "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "tied_lm_head": bool(cfg["tie_word_embeddings"]),
                   "prompt_len": list(wl["prompt_len"]), "output_len": list(wl["output_len"]),
                   "arrivals": f"Poisson, {wl['arrival_rate']}/s" if wl["arrival_rate"] > 0 else "all at once",
                   "context_len": wl["context_len"], "page_size": PAGE_SIZE, "max_num_seqs": wl["max_num_seqs"],
                   "tokens_per_step": PREFILL_TOKENS, "pool_pages": num_pages, "pool_gb": round(kv_bytes / 1e9, 2),
                   "all_resident_gb": round(kv_bytes / num_pages / PAGE_SIZE * need_tokens / 1e9, 2), "seed": seed},
    }
    log(f"  {res['value']:.0f} output tok/s in {seconds:.2f} s, {st['steps']} steps, TTFT p50 {res['ttft_ms']['p50']:.0f} ms, "
        f"per token p50 {res['per_token_ms']['p50']:.2f} ms, {st['preemptions']} preemptions "
        f"({st['recomputed_tokens']} tokens recomputed)")
    del eng, llm
    gc.collect()
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="skip batch 1 / 64 and the prefill measurement")
    ap.add_argument("--check", action="store_true",
                    help="also compare logits of a 2-layer model of these widths with the plain implementation under "
                         "tests/ on the timed paths (adds about a minute); the line gets a \"check\" key and the exit "
                         "code is 1 if the limit is broken")
    ap.add_argument("--workload", default="all", choices=["all", "none", *WORKLOADS],
                    help="the serving workloads measured beside the headline (3B continuous batching, 8B under a "
                         "pool that is too small); one name runs that workload alone and prints its own JSON line")
    args = ap.parse_args()

    if args.impl == "reference":
        # upstream's own engine, unmodified, driven through its standard input and output
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        return reference_arm.run(args, dict(LLAMA_1B), PROMPT_LEN, NEW_TOKENS, ClockSampler)
    if args.gpus != 1:
        print(f"bench.py measures one GPU only (this engine runs on one GPU); got --gpus {args.gpus}")
        return 2
    if args.steps < 1 or args.warmup < 3 or args.steps + args.warmup + 2 > NEW_TOKENS:
        print(f"need steps >= 1, warmup >= 3 and steps + warmup + 2 <= {NEW_TOKENS}")
        return 2

    import torch
    from kv_cache_optimization_for_llm_b200 import LLM

    if args.workload in WORKLOADS:
        print(json.dumps({"workload": args.workload, **run_workload(args.workload)}), flush=True)
        return 0
    cfg = dict(LLAMA_1B)
    cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    nums = model_numbers(cfg, args.layers)
    max_batch = max(args.batch, 1 if args.skip_points else 64)
    log(f"building Llama-3.2-1B shape, {args.layers} layers, random bfloat16 weights")
    llm = LLM.from_random(cfg, seed=0, std=0.02, dtype="bfloat16", page_size=PAGE_SIZE,
                          num_pages=max_batch * (CONTEXT_LEN // PAGE_SIZE) // 4 + PREFILL_TOKENS // PAGE_SIZE,
                          max_num_seqs=max_batch, max_num_batched_tokens=PREFILL_TOKENS, max_model_len=CONTEXT_LEN)
    sampler = ClockSampler()
    sampler.start()
    windows = []

    log(f"decode, batch {args.batch}: device-timed")
    sec, mean_ctx, launches, win = run_decode(llm, args.batch, args.steps, args.warmup, False, seed=1)
    windows.append(win)
    value = args.batch * args.steps / sec
    ms_per_step = 1000.0 * sec / args.steps
    log(f"  {value:.0f} tok/s, {ms_per_step:.3f} ms/step, {launches} launches")
    log(f"decode, batch {args.batch}: end to end")
    sec_e, _, _, win = run_decode(llm, args.batch, args.steps, args.warmup, True, seed=1)
    windows.append(win)
    e2e = args.batch * args.steps / sec_e
    b_in = run_decode.h2d_bytes + 4 * 4 * args.batch   # batch arrays + sampler parameters
    log(f"  {e2e:.0f} tok/s")

    step_bytes = nums["weight_bytes"] + args.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1000.0) / 1e9
    points, point_rooflines, prefill = {}, {}, None
    if not args.skip_points:
        for b in (1, 64):
            log(f"decode, batch {b}")
            s, ctx_b, _, win = run_decode(llm, b, args.steps, args.warmup, False, seed=2 + b)
            windows.append(win)
            points[f"decode_b{b}"] = round(b * args.steps / s, 1)
            bytes_b = nums["weight_bytes"] + b * ctx_b * nums["kv_bytes_per_token"]
            gbs = bytes_b / (s / args.steps) / 1e9
            point_rooflines[f"decode_b{b}"] = {"ms_per_step": round(1000.0 * s / args.steps, 4), "bytes": int(bytes_b),
                                               "achieved": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}
            log(f"  {points[f'decode_b{b}']:.0f} tok/s, {gbs:.0f} GB/s = {gbs / pk['hbm_gbs']:.3f} of {pk['source']} HBM peak")
        log(f"prefill of {PREFILL_TOKENS} tokens")
        w0 = time.perf_counter()
        ms = run_prefill(llm, reps=5, warmup=3, seed=9)
        windows.append((w0, time.perf_counter()))
        fl = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / (ms / 1000.0), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                   "frac": round(fl / (ms / 1000.0) / (pk["bf16_tflops"] * 1e12), 4)}
        log(f"  {prefill['value']:.0f} tok/s, {ms:.2f} ms, {prefill['frac']:.3f} of {pk['source']} bf16 peak")
        log("time to the first token of a lone 128-token prompt")
        w0 = time.perf_counter()
        points["first_token_ms_prompt128"] = round(run_first_token(llm, 128, reps=7, warmup=3, seed=13), 3)
        windows.append((w0, time.perf_counter()))
        log(f"  {points['first_token_ms_prompt128']:.2f} ms")
    sampler.stop()
    clocks = sampler.summary(windows)
    b_out = 4 * args.batch + 4                                              # sampled ids + the status word
    graphs_on = bool(llm.engine.config.use_cuda_graphs)
    workloads = {}
    if args.workload == "all" and not args.skip_points:
        del llm
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for name in WORKLOADS:
            try:
                workloads[name] = run_workload(name)
            except Exception as e:       # the headline must not be lost to a side measurement
                workloads[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                log(f"{name} failed: {workloads[name]['error']}")

    line = {
        "metric": "decode tok/s (Llama-3.2-1B shape, bf16, batch 8, 512-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02)",
        "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B shape (LlamaForCausalLM)", "layers": args.layers, "layers_full_model": FULL_LAYERS,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"], "tied_lm_head": True,
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "new_tokens": NEW_TOKENS,
            "context_len": CONTEXT_LEN, "page_size": PAGE_SIZE, "kv_dtype": "bf16", "parallelism": "none (1 GPU)",
            "l2": "inputs larger than L2: 2.47 GB of weights are streamed every step",
            "cuda_graphs": graphs_on,
        },
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(b_in),
                "d2h_bytes_per_step": int(b_out)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"], "bytes": int(step_bytes),
                     "points": point_rooflines},
        "clocks": clocks,
    }
    if prefill is not None:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    if workloads:
        line["workloads"] = workloads
    if args.check:
        log("logits of a 2-layer model of these widths against the plain implementation")
        line["check"] = run_value_check(dict(LLAMA_1B))
        log(f"  {line['check']}")
    print(json.dumps(line), flush=True)
    return 0 if not args.check or line["check"]["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())

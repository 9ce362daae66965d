"""Command line of the engine, in upstream's manner.

    python -m kv_cache_optimization_for_llm_b200.cli [MODEL_DIR] [options] < requests

The model folder is the positional argument or ``MODEL_DIR``; sampling is set by
``TEMPERATURE``, ``SAMPLING_SEED`` and ``IGNORE_EOS=1`` (flags of the same meaning
override them); ``PREEMPTION_POLICY`` accepts ``recompute`` only
(base/src/main.cu:42-104, paged_attention/src/main.cu:67-92).

Requests arrive on standard input, one per line, as upstream's wire format
(base/src/request_queue.cpp:11-61):

    <request_id> <max_tokens> <n_seqs> <token> <token> ...

and answers leave on standard output as JSON lines with upstream's fields: one
``engine_config`` line, ``{"id","slot","seq","tok"}`` per generated token,
``{"type":"preempted",...}`` when a request is sent back to the queue, and
``{"id","slot","seq","done":true,"tokens","decode_time","decode_speed"[,"error"]}``
when a request ends (base/src/engine.cu:389-408,472-484,933-940).  Token ids only:
text belongs to the client.  The process ends when its input is closed and every
request has finished.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import threading
import time
from collections import deque


def _parse_line(line: str):
    parts = line.split()
    if len(parts) < 4:
        raise ValueError("a request line needs: id max_tokens n_seqs token...")
    rid, max_tokens, n_seqs = int(parts[0]), int(parts[1]), int(parts[2])
    if max_tokens < 1:
        raise ValueError(f"request {rid} has no usable output budget")
    if not 1 <= n_seqs <= 8:
        raise ValueError(f"request {rid}: n_seqs is {n_seqs}, outside 1..8")
    return rid, max_tokens, n_seqs, [int(t) for t in parts[3:]]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kv_cache_optimization_for_llm_b200.cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_dir", nargs="?", default=os.environ.get("MODEL_DIR"),
                    help="folder with config.json and model.safetensors (or MODEL_DIR)")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="write a random-weights model for this config.json "
                    "into a temporary folder and serve it")
    ap.add_argument("--seed", type=int, default=0, help="seed of --random weights")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--temperature", type=float, default=None, help="overrides TEMPERATURE (0: greedy)")
    ap.add_argument("--sampling-seed", type=int, default=None, help="overrides SAMPLING_SEED")
    ap.add_argument("--ignore-eos", action="store_true", help="same as IGNORE_EOS=1")
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--prompt-ids", help="one request given on the command line: token ids separated by spaces")
    ap.add_argument("--max-tokens", type=int, default=64, help="output budget of --prompt-ids")
    ap.add_argument("--telemetry-every", type=int, default=0, help="emit a 'step' line every N steps (upstream: 8)")
    args = ap.parse_args(argv)

    temperature = args.temperature if args.temperature is not None else max(0.0, float(os.environ.get("TEMPERATURE", "0") or 0))
    seed = args.sampling_seed if args.sampling_seed is not None else int(os.environ.get("SAMPLING_SEED", "0") or 0)
    ignore_eos = args.ignore_eos or os.environ.get("IGNORE_EOS", "")[:1] == "1"
    policy = os.environ.get("PREEMPTION_POLICY", "recompute")
    if policy != "recompute":
        print(f'PREEMPTION_POLICY must be "recompute" (swapping pages to host memory is not built), got "{policy}"',
              file=sys.stderr)
        return 1

    from . import EngineConfig, SamplingParams
    from .engine.llm_engine import LLMEngine
    from .weights import write_random_model

    model_dir = args.model_dir
    if args.random:
        with open(args.random) as f:
            cfg_dict = json.load(f)
        model_dir = tempfile.mkdtemp(prefix="kvb200_random_")
        write_random_model(model_dir, cfg_dict, args.seed,
                           storage_dtype="float32" if args.dtype in ("float32", "fp32") else "bfloat16")
    if not model_dir:
        print("no model: give a model folder, MODEL_DIR, or --random CONFIG_JSON", file=sys.stderr)
        return 1
    print(f"Model directory: {model_dir}", file=sys.stderr)
    if temperature > 0:
        print(f"Sampling: temperature {temperature}, seed {seed} (greedy decoding is OFF)", file=sys.stderr)

    engine = LLMEngine(model_dir, EngineConfig(
        dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages, max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len, seed=seed))
    m = engine.runner.manager

    def emit(obj):
        sys.stdout.write(json.dumps(obj) + "\n")
        sys.stdout.flush()

    emit({"type": "engine_config", "mechanism": "paged", "batch_size": args.max_num_seqs,
          "max_batch_tokens": args.max_num_batched_tokens, "max_model_len": engine.runner.max_model_len,
          "block_size": args.page_size, "kv_pool_tokens": m.num_pages(0) * args.page_size,
          "temperature": temperature, "sampling_seed": seed, "preemption_policy": "recompute",
          "dtype": engine.config.dtype})

    pending = deque()
    lock = threading.Lock()
    closed = threading.Event()

    def reader():
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            try:
                req = _parse_line(line)
            except ValueError as e:
                print(f"Malformed input line, ignoring: {e}", file=sys.stderr)
                continue
            with lock:
                pending.append(req)
        closed.set()

    if args.prompt_ids:
        pending.append((0, args.max_tokens, 1, [int(t) for t in args.prompt_ids.split()]))
        closed.set()
    else:
        threading.Thread(target=reader, daemon=True).start()

    meta = {}       # engine id -> (wire id, seq, n generated, decode start)
    steps = 0
    t_start = time.perf_counter()
    total_tokens = 0
    while True:
        with lock:
            new = list(pending)
            pending.clear()
        for rid, max_tokens, n_seqs, tokens in new:
            for seq in range(n_seqs):
                sp = SamplingParams(max_tokens=max_tokens, temperature=temperature, ignore_eos=ignore_eos,
                                    repetition_penalty=args.repetition_penalty)
                try:
                    eid = engine.add_request(tokens, sp, key=rid * 8 + seq)   # upstream's stream key
                except ValueError as e:
                    emit({"id": rid, "slot": -1, "seq": seq, "done": True, "tokens": 0, "decode_time": 0.0,
                          "decode_speed": 0.0, "error": str(e)})
                    continue
                meta[eid] = [rid, seq, 0, None]
        if not engine.has_unfinished():
            if closed.is_set():
                with lock:
                    if not pending:
                        break
            time.sleep(0.005)   # upstream sleeps 5 ms when idle (base/src/main.cu:166)
            continue
        before = engine.stats()["preemptions"]
        events = engine.step()
        steps += 1
        now = time.perf_counter()
        if engine.stats()["preemptions"] > before:
            emit({"type": "preempted", "policy": "recompute", "count": engine.stats()["preemptions"] - before})
        for ev in events:
            info = meta.get(ev.request_id)
            if info is None:
                continue
            if ev.token is not None:
                if info[3] is None:
                    info[3] = now
                info[2] += 1
                total_tokens += 1
                emit({"id": info[0], "slot": ev.slot, "seq": info[1], "tok": ev.token})
            if ev.finished:
                ms = (now - info[3]) * 1000.0 if info[3] is not None else 0.0
                done = {"id": info[0], "slot": ev.slot, "seq": info[1], "done": True, "tokens": info[2],
                        "decode_time": ms, "decode_speed": (info[2] / (ms / 1000.0)) if ms > 0 else 0.0}
                if ev.reason not in ("stop", "length"):
                    done["error"] = ev.reason
                emit(done)
                meta.pop(ev.request_id, None)
        if args.telemetry_every and steps % args.telemetry_every == 0:
            s = engine.stats()
            emit({"type": "step", "step": steps, "running": s["running"], "waiting": s["waiting"],
                  "kv_total_pages": s["num_pages"][0], "kv_free_pages": s["free_pages"][0],
                  "preemptions": s["preemptions"]})
    dt = time.perf_counter() - t_start
    print(f"{total_tokens} tokens in {steps} steps, {dt:.2f} s ({total_tokens / dt if dt > 0 else 0:.1f} tok/s overall)",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())

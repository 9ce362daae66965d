"""The reference arm of bench.py: upstream's paged engine, unmodified, on the same workload.

Upstream (thientd05/kv_cache_optimization_for_llm, paged_attention/) is a CUDA program that
reads requests from standard input, ``<id> <max_tokens> <n_seqs> <token ids...>`` a line
(paged_attention/src/request_queue.cpp:11-61), and writes one JSON line per generated token
to standard output (paged_attention/src/engine.cu:1817-1827); its own benchmark drives it the
same way, as a child process with ``IGNORE_EOS=1`` (bench.py:120-137).  Its sources are
copied as they are into ``baseline/_ref/paged_attention`` and compiled with the flags of its
CMakeLists.txt, the architecture set to sm_100a on the command line.  Its sizes are
compile-time constants for exactly the benchmark's model (Llama-3.2-1B,
paged_attention/src/config.h:43-54), and its loader takes tensors by name without looking at
their values, so the random bfloat16 model folder that this package writes is what it loads.

One thing has to be arranged around it.  Its decode attention forms a page's byte offset as
``int * int`` (paged_attention/src/kernels.cu:175-176: ``physical_block * BLOCK_BYTES``, 32 KiB
a page), which overflows from page 65 536 on, and its pool is "whatever memory is free"
(paged_attention/src/engine.cu:194-215), handed out from the highest page down.  It was
written for a 4 GB card; on a 180 GB one the first request would already read far outside
the pool.  So this process holds device memory of its own while the engine starts, enough
that the pool comes out just under 65 536 pages (2 GiB, 60 000 tokens of context: room for
64 requests of 768 tokens), checks the page count that the engine reports before any request
is sent, and gives up if it is larger.

The 2048-token prompt of the prefill point exceeds upstream's MAX_PROMPT_LEN = 1024
(paged_attention/src/config.h:81), so that point has no reference number.
"""

from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref", "paged_attention")
BINARY = os.path.join(REF_DIR, "tiny-vllm")
SOURCES = ["main.cu", "engine.cu", "kernels.cu", "model.cu", "utils.cu", "request_queue.cpp"]
UPSTREAM = os.path.join(os.environ.get("KVB200_UPSTREAM_DIR", "/root/reference"), "paged_attention")   # where upstream is checked out
PAGE_BYTES = 32 * 1024          # BLOCK_BYTES: 16 tokens x 512 x bfloat16 x (K and V), one layer
MAX_SAFE_PAGES = 65535          # the largest page count whose int offsets do not overflow
TARGET_PAGES = 61000
MAX_PROMPT_LEN = 1024


class Unavailable(RuntimeError):
    pass


def log(msg):
    print(f"[bench reference] {msg}", file=sys.stderr, flush=True)


def ensure_built():
    """The unmodified sources under baseline/_ref, compiled for sm_100a if the binary is not there."""
    if not os.path.isdir(os.path.join(REF_DIR, "src")):
        if not os.path.isdir(UPSTREAM):
            raise Unavailable("upstream's sources are neither under baseline/_ref/paged_attention nor at " + UPSTREAM)
        os.makedirs(os.path.dirname(REF_DIR), exist_ok=True)
        shutil.copytree(UPSTREAM, REF_DIR)
    if os.path.exists(BINARY):
        return
    nvcc = os.environ.get("KVB200_NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Isrc", "-Iinclude",
           *[os.path.join("src", s) for s in SOURCES], "-lcublas", "-o", "tiny-vllm"]
    log("compiling upstream's paged engine for sm_100a (about a minute)")
    r = subprocess.run(cmd, cwd=REF_DIR, capture_output=True, text=True)
    if r.returncode != 0 or not os.path.exists(BINARY):
        raise Unavailable("upstream's sources did not compile for sm_100a: " + (r.stderr.strip().splitlines() or ["?"])[-1])


class Engine:
    """The engine as a child process; a thread stamps every line it writes."""

    def __init__(self, model_dir, log_path):
        env = dict(os.environ)
        env["IGNORE_EOS"] = "1"
        env.pop("TEMPERATURE", None)
        self.err = open(log_path, "w")
        self.proc = subprocess.Popen([BINARY, model_dir], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                     stderr=self.err, text=True, bufsize=1, env=env, cwd=REF_DIR)
        self.lines = []          # (time, parsed JSON)
        self.lock = threading.Lock()
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            t = time.perf_counter()
            try:
                d = json.loads(line)
            except ValueError:
                continue
            with self.lock:
                self.lines.append((t, d))

    def wait_for(self, pred, timeout, what):
        """The first line (from the start) for which ``pred`` holds."""
        t_end = time.perf_counter() + timeout
        seen = 0
        while True:
            with self.lock:
                new = self.lines[seen:]
                seen = len(self.lines)
            for t, d in new:
                if pred(d):
                    return t, d
            if self.proc.poll() is not None:
                raise Unavailable(f"upstream's engine exited with code {self.proc.returncode} while {what}")
            if time.perf_counter() > t_end:
                raise Unavailable(f"upstream's engine did not answer within {timeout:.0f} s while {what}")
            time.sleep(0.005)

    def send(self, text):
        self.proc.stdin.write(text)
        self.proc.stdin.flush()

    def snapshot(self):
        with self.lock:
            return list(self.lines)

    def stop(self):
        """Ends exactly this child (it serves forever by design: paged_attention/src/main.cu:133)."""
        if self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait(timeout=10)
        self.err.close()


def hold_memory(torch, leave_free_bytes, held):
    """Allocates device memory in this process until about ``leave_free_bytes`` stay free."""
    free, _ = torch.cuda.mem_get_info()
    want = free - int(leave_free_bytes)
    chunk = 8 << 30
    while want > (64 << 20):
        n = min(chunk, want)
        held.append(torch.empty(n, dtype=torch.uint8, device="cuda"))
        want -= n
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def start_engine_with_a_pool_that_fits(torch, model_dir, log_dir):
    """Starts the engine twice if needed: once to learn how large its pool comes out with
    8 GB left free, then with this process holding the difference.  Returns (engine, pages)."""
    held = []
    free = hold_memory(torch, 8 << 30, held)
    log(f"holding device memory so that {free / 2**30:.1f} GiB stay free for upstream's engine")
    for attempt in range(3):
        eng = Engine(model_dir, os.path.join(log_dir, f"engine_{attempt}.log"))
        try:
            _, cfg = eng.wait_for(lambda d: d.get("type") == "engine_config", 300, "loading the model")
        except Unavailable:
            eng.stop()
            raise
        pages = int(cfg["num_blocks"])
        log(f"upstream's pool: {pages} pages = {cfg.get('kv_pool_tokens')} tokens of context")
        if pages <= MAX_SAFE_PAGES:
            return eng, pages, held
        eng.stop()       # nothing was sent, so no kernel has touched the pool
        excess = (pages - TARGET_PAGES) * PAGE_BYTES
        free = hold_memory(torch, torch.cuda.mem_get_info()[0] - excess, held)
        log(f"too many pages for its 32-bit page offsets; holding {excess / 2**30:.2f} GiB more")
    raise Unavailable("upstream's pool could not be brought under 65 536 pages (its int page offsets overflow beyond)")


def request_lines(ids, prompts, max_tokens):
    return "".join(f"{i} {max_tokens} 1 {' '.join(map(str, p))}\n" for i, p in zip(ids, prompts))


def measure_decode(eng, batch, steps, warmup, prompt_len, new_tokens, vocab, seed, first_id):
    """Sends ``batch`` requests at once and times ``steps`` decode steps in which all of them run.
    Returns a dict with tokens a second and ms per step, measured on the lines as they arrive."""
    import numpy as np
    rng = np.random.default_rng(seed)
    ids = list(range(first_id, first_id + batch))
    prompts = [rng.integers(0, vocab, prompt_len).tolist() for _ in ids]
    base = len(eng.snapshot())
    t_sent = time.perf_counter()
    eng.send(request_lines(ids, prompts, new_tokens))
    done = set()

    def finished(d):
        if d.get("done") and d.get("id") in ids:
            done.add(d["id"])
        return len(done) == batch
    eng.wait_for(finished, 600, f"decoding at batch {batch}")
    lines = eng.snapshot()[base:]
    toks = {i: [] for i in ids}
    errors = [d for _, d in lines if d.get("done") and d.get("error")]
    if errors:
        raise Unavailable(f"upstream's engine ended a request with an error at batch {batch}: {errors[0].get('error')}")
    for t, d in lines:
        if "tok" in d and d.get("id") in toks:
            toks[d["id"]].append(t)
    counts = {i: len(v) for i, v in toks.items()}
    if any(c != new_tokens for c in counts.values()):
        raise Unavailable(f"upstream's engine emitted {sorted(set(counts.values()))} tokens per request, not {new_tokens}")
    # the request whose first token came last: from then on every step carries all of them
    last = max(ids, key=lambda i: toks[i][0])
    first_done = min(v[-1] for v in toks.values())
    stamps = toks[last]
    if warmup + steps >= len(stamps):
        raise Unavailable(f"{warmup} + {steps} steps do not fit into {len(stamps)} decode steps")
    t0, t1 = stamps[warmup], stamps[warmup + steps]
    if t1 > first_done:
        raise Unavailable("a request finished inside the timed steps")
    n = sum(1 for v in toks.values() for t in v if t0 < t <= t1)
    ttft = max(v[0] for v in toks.values()) - t_sent
    reported = [d for _, d in lines if d.get("done")]
    own = sum(d["tokens"] for d in reported) / (max(d["decode_time"] for d in reported) / 1000.0)
    return {"value": n / (t1 - t0), "ms_per_step": 1000.0 * (t1 - t0) / steps, "tokens": n, "expected": batch * steps,
            "window": (t0, t1), "prompts_read_s": ttft, "upstream_decode_speed": own}


def measure_prefill_1024(eng, vocab, seed, rid):
    """Upstream's own figure for one packed pass over a 1024-token prompt (its longest)."""
    import numpy as np
    prompt = np.random.default_rng(seed).integers(0, vocab, MAX_PROMPT_LEN).tolist()
    out = None
    for k in range(3):           # the first passes warm up
        base = len(eng.snapshot())
        eng.send(request_lines([rid + k], [prompt], 1))
        eng.wait_for(lambda d, k=k: d.get("done") and d.get("id") == rid + k, 120, "reading a 1024-token prompt")
        for _, d in eng.snapshot()[base:]:
            if d.get("type") == "prefill_stats" and d.get("id") == rid + k:
                out = d
    if out is None:
        return None
    return {"tokens": int(out["batch_tokens"]), "ms": round(float(out["time_ms"]), 3),
            "value": round(float(out["speed"]), 1), "timed_by": "upstream's own prefill_stats line"}


def run(args, model_config, prompt_len, new_tokens, clock_sampler_cls):
    """Prints the reference arm's JSON line.  Returns the exit code."""
    line = {"impl": "reference"}
    tmp = None
    eng = None
    try:
        if args.gpus != 1:
            print(f"bench.py measures one GPU only (upstream runs on one GPU); got --gpus {args.gpus}")
            return 2
        ensure_built()
        import torch
        if not torch.cuda.is_available():
            raise Unavailable("no CUDA device is visible")
        sys.path.insert(0, os.path.dirname(HERE))
        from kv_cache_optimization_for_llm_b200.weights import write_random_model
        tmp = tempfile.mkdtemp(prefix="kvb200_refarm_")
        log("writing the random bfloat16 model folder (2.5 GB)")
        model_dir = write_random_model(os.path.join(tmp, "model"), model_config, seed=0, std=0.02,
                                       storage_dtype="bfloat16")
        torch.cuda.init()
        eng, pages, held = start_engine_with_a_pool_that_fits(torch, str(model_dir), tmp)
        vocab = model_config["vocab_size"]
        steps = min(args.steps, new_tokens - args.warmup - 8)
        sampler = clock_sampler_cls()
        sampler.start()
        log("warm-up: one request")
        measure_decode(eng, 1, 8, 3, prompt_len, 32, vocab, seed=99, first_id=9000)
        results = {}
        for b, first in ((args.batch, 100), (1, 1000), (64, 2000)):
            if b in results:
                continue
            log(f"decode, batch {b}")
            results[b] = measure_decode(eng, b, steps, args.warmup, prompt_len, new_tokens, vocab, seed=1 + b, first_id=first)
            r = results[b]
            log(f"  {r['value']:.0f} tok/s, {r['ms_per_step']:.3f} ms/step ({r['tokens']} of {r['expected']} tokens in the window; "
                f"upstream's own decode_speed sums to {r['upstream_decode_speed']:.0f} tok/s)")
        prefill_1024 = measure_prefill_1024(eng, vocab, seed=9, rid=5000)
        sampler.stop()
        head = results[args.batch]
        line.update({
            "metric": "decode tok/s (Llama-3.2-1B shape, bf16, batch 8, 512-token prompts)",
            "value": round(head["value"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
            "ms_per_step": round(head["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform-random token ids, random-init weights N(0,0.02)",
            "config": {
                "model": "Llama-3.2-1B shape (upstream's compile-time sizes)", "layers": model_config["num_hidden_layers"],
                "layers_full_model": model_config["num_hidden_layers"], "hidden_size": model_config["hidden_size"],
                "intermediate_size": model_config["intermediate_size"],
                "num_attention_heads": model_config["num_attention_heads"],
                "num_key_value_heads": model_config["num_key_value_heads"], "head_dim": model_config["head_dim"],
                "vocab_size": vocab, "tied_lm_head": True, "global_batch": args.batch, "prompt_len": prompt_len,
                "new_tokens": new_tokens, "context_len": 2048, "page_size": 16, "kv_dtype": "bf16",
                "parallelism": "none (1 GPU)", "kv_pool_pages": pages,
                "timing": "wall clock on the token lines of upstream's standard output (its only interface)",
            },
            "e2e": {"value": round(head["value"], 1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                    "d2h_bytes_per_step": None, "note": "token ids in through standard input, out through standard output"},
            "points": {f"decode_b{b}": round(r["value"], 1) for b, r in results.items() if b != args.batch},
            "prefill": {"unavailable": f"a 2048-token prompt exceeds upstream's MAX_PROMPT_LEN = {MAX_PROMPT_LEN}",
                        "same_config": False, "prompt_1024": prefill_1024},
            "clocks": sampler.summary([r["window"] for r in results.values()]),
        })
    except Unavailable as e:
        line = {"impl": "reference", "unavailable": str(e)}
    finally:
        if eng is not None:
            eng.stop()
        if tmp is not None:
            shutil.rmtree(tmp, ignore_errors=True)
    print(json.dumps(line), flush=True)
    return 0

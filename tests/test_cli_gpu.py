"""The command line in upstream's manner: the model folder as argument or MODEL_DIR,
requests as "<id> <max_tokens> <n_seqs> <token>..." lines on standard input, answers as
JSON lines with upstream's fields; TEMPERATURE / SAMPLING_SEED / IGNORE_EOS as upstream
reads them."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as P
from tiny_models import model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(args, lines, env=None):
    e = dict(os.environ)
    e.update(env or {})
    e["PYTHONPATH"] = ROOT + os.pathsep + e.get("PYTHONPATH", "")
    p = subprocess.run([sys.executable, "-m", "kv_cache_optimization_for_llm_b200.cli", *args],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, env=e, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    return [json.loads(l) for l in p.stdout.splitlines() if l.strip()], p.stderr


def test_wire_format_greedy_and_sampled():
    mdir = model_dir("tiny_a", "float32")
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(3)
    prompts = {7: rng.integers(0, 250, 6).tolist(), 12: rng.integers(0, 250, 15).tolist()}
    lines = [f"{rid} 5 1 " + " ".join(map(str, toks)) for rid, toks in prompts.items()]
    lines.append("garbage line")                     # ignored with a message, as upstream does
    out, err = run_cli([mdir, "--dtype", "float32", "--page-size", "4", "--num-pages", "64", "--max-num-seqs", "4"],
                       lines, env={"IGNORE_EOS": "1"})
    assert "Malformed input line" in err
    assert out[0]["type"] == "engine_config" and out[0]["mechanism"] == "paged" and out[0]["block_size"] == 4
    toks = {rid: [m["tok"] for m in out if m.get("id") == rid and "tok" in m] for rid in prompts}
    done = {m["id"]: m for m in out if m.get("done")}
    for rid, prompt in prompts.items():
        assert toks[rid] == P.generate(cfg, w, prompt, 5)
        assert done[rid]["tokens"] == 5 and done[rid]["seq"] == 0 and "error" not in done[rid]
    # TEMPERATURE and SAMPLING_SEED from the environment; n_seqs = 2 gives two independent
    # sequences whose random streams are keyed id*8+seq, as upstream's are
    out, _ = run_cli(["--dtype", "float32", "--page-size", "4", "--num-pages", "64"],
                     ["3 4 2 " + " ".join(map(str, prompts[7]))],
                     env={"MODEL_DIR": mdir, "TEMPERATURE": "0.8", "SAMPLING_SEED": "5", "IGNORE_EOS": "1"})
    assert out[0]["temperature"] == 0.8 and out[0]["sampling_seed"] == 5
    for seq in (0, 1):
        got = [m["tok"] for m in out if m.get("id") == 3 and m.get("seq") == seq and "tok" in m]
        assert got == P.generate(cfg, w, prompts[7], 4, temperature=0.8, seed=5, key=3 * 8 + seq)


def test_swap_policy_is_refused_and_prompt_ids_flag_works():
    mdir = model_dir("tiny_a", "float32")
    e = dict(os.environ, PREEMPTION_POLICY="swap", PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-m", "kv_cache_optimization_for_llm_b200.cli", mdir], input="",
                       capture_output=True, text=True, env=e, timeout=300)
    assert p.returncode == 1 and "recompute" in p.stderr
    cfg, w = P.read_model_dir(mdir)
    out, _ = run_cli([mdir, "--dtype", "float32", "--page-size", "4", "--num-pages", "32", "--prompt-ids", "5 6 7 8",
                      "--max-tokens", "3", "--ignore-eos"], [])
    assert [m["tok"] for m in out if "tok" in m] == P.generate(cfg, w, [5, 6, 7, 8], 3)

"""The harness around upstream's engine (baseline/reference_arm.py), against a stand-in that
speaks upstream's wire format on the CPU: request lines in, an ``engine_config`` line, one
JSON line per token, ``prefill_stats`` and ``done`` lines out
(paged_attention/src/request_queue.cpp:11-61, engine.cu:256-292,408-425,1395-1460,1817-1849).
What is checked is the harness's own arithmetic: which steps it times, that it counts exactly
batch x steps tokens in the window, and what it refuses."""

import os
import stat
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

FAKE = textwrap.dedent('''\
    #!%s
    import json, sys, threading, time, collections
    STEP = float(sys.argv[2]) if len(sys.argv) > 2 else 0.004
    print(json.dumps({"type": "engine_config", "num_blocks": int(sys.argv[3]) if len(sys.argv) > 3 else 60000,
                      "kv_pool_tokens": 60000}), flush=True)
    queue, lock = collections.deque(), threading.Lock()
    def reader():
        for line in sys.stdin:
            f = line.split()
            if len(f) < 4: continue
            with lock: queue.append((int(f[0]), int(f[1]), len(f) - 3))
    threading.Thread(target=reader, daemon=True).start()
    live = {}      # id -> [remaining, produced, t_start]
    while True:
        with lock:
            new = [queue.popleft() for _ in range(len(queue))]
        for rid, budget, plen in new:           # "prefill": the first token
            print(json.dumps({"id": rid, "slot": 0, "seq": 0, "tok": 7}), flush=True)
            print(json.dumps({"type": "prefill_stats", "id": rid, "speed": 1000.0, "time_ms": 1.0,
                              "prompt_tokens": plen, "batch_tokens": plen, "batch_prompts": 1, "resumed_tokens": 0}), flush=True)
            live[rid] = [budget - 1, 1, time.time()]
            if budget == 1:
                print(json.dumps({"id": rid, "done": True, "tokens": 1, "decode_time": 1.0, "decode_speed": 1.0}), flush=True)
                del live[rid]
        if not live:
            time.sleep(0.001); continue
        time.sleep(STEP)                         # one decode step for everybody
        for rid in sorted(live):
            st = live[rid]
            print(json.dumps({"id": rid, "slot": 0, "seq": 0, "tok": 9}), flush=True)
            st[0] -= 1; st[1] += 1
            if st[0] == 0:
                ms = 1000.0 * (time.time() - st[2])
                print(json.dumps({"id": rid, "done": True, "tokens": st[1], "decode_time": ms,
                                  "decode_speed": st[1] / (ms / 1000.0)}), flush=True)
                del live[rid]
    ''') % sys.executable


@pytest.fixture()
def arm(tmp_path, monkeypatch):
    import reference_arm as R
    fake = tmp_path / "tiny-vllm"
    fake.write_text(FAKE)
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setattr(R, "BINARY", str(fake))
    monkeypatch.setattr(R, "REF_DIR", str(tmp_path))
    return R, tmp_path


def test_decode_window_counts_batch_times_steps_tokens(arm):
    R, tmp = arm
    eng = R.Engine("unused-model-dir", str(tmp / "engine.log"))
    try:
        _, cfg = eng.wait_for(lambda d: d.get("type") == "engine_config", 20, "starting")
        assert cfg["num_blocks"] == 60000
        res = R.measure_decode(eng, batch=4, steps=10, warmup=3, prompt_len=8, new_tokens=32, vocab=100, seed=1, first_id=100)
        assert res["tokens"] == res["expected"] == 40
        # four tokens per step of about 4 ms (the stand-in sleeps; the host adds its own time)
        assert 2.5 < res["ms_per_step"] < 12.0
        assert abs(res["value"] - 4 / (res["ms_per_step"] / 1000.0)) < 1e-6 * res["value"] + 1e-3
        one = R.measure_decode(eng, batch=1, steps=5, warmup=3, prompt_len=4, new_tokens=16, vocab=100, seed=2, first_id=200)
        assert one["tokens"] == 5
        # too many steps for the budget is refused, not mis-measured
        with pytest.raises(R.Unavailable, match="do not fit"):
            R.measure_decode(eng, batch=2, steps=20, warmup=5, prompt_len=4, new_tokens=16, vocab=100, seed=3, first_id=300)
        pre = R.measure_prefill_1024(eng, vocab=100, seed=4, rid=400)
        assert pre["tokens"] == 1024 and pre["value"] == 1000.0
    finally:
        eng.stop()
    assert eng.proc.poll() is not None          # exactly this child was ended

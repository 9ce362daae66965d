"""What bench.py promises its caller that needs no GPU: one line and exit code 2 for more than one GPU, the
limits on its step counts, and the bytes and FLOPs that its roofline fractions are counted from."""

import os
import sys


def _bench_module():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    return bench


def test_bench_refuses_more_than_one_gpu_with_one_line_and_exit_code_2():
    import subprocess
    root = os.path.dirname(os.path.dirname(__file__))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
    # too few warm-up steps are refused as well (the timing rules want at least three)
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--steps", "4", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "warmup" in r.stdout


def test_bench_counts_the_bytes_and_flops_of_the_named_shape():
    """The roofline's numerators: every weight once (the tied head's matrix counted once), keys and values of
    one token in every layer, and the FLOPs of a prefill with causal attention."""
    bench = _bench_module()
    cfg = dict(bench.LLAMA_1B)
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    n = bench.model_numbers(cfg, L)
    per_layer = H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I + 2 * H
    assert n["weight_bytes"] == 2 * (V * H + L * per_layer + H)
    assert n["kv_bytes_per_token"] == 2 * 2 * L * nkv * d
    assert abs(n["weight_bytes"] / 1e9 - 2.47) < 0.01        # the 2.47 GB that the config line names
    T = 2048
    fl = bench.prefill_flops(cfg, L, T)
    products = 2 * T * L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    assert products < fl < products * 1.2                     # attention and the head on top of the products
    half = bench.model_numbers(cfg, L // 2)
    assert half["weight_bytes"] == 2 * (V * H + (L // 2) * per_layer + H)

"""Drives bin/trace_run as a user would: a child process, steps on its standard
input, one ``done <step>`` line back per step, logits read from the output folder."""

import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def ceil64(n):
    return -(-n // 64) * 64


class TraceRun:
    def __init__(self, model, dtype, max_tokens, extra=()):
        self.out = tempfile.mkdtemp(prefix="kvb200_trace_")
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype,
               "--out", self.out, "--max-tokens", str(max_tokens), *extra]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want).  Returns the logits [wanted, vocab] or None."""
        msg = {"step": self.step_no,
               "entries": [{"id": i, "tokens": list(map(int, t)), "want": list(map(int, w))} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(msg) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            rc = self.proc.poll()
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_no} (exit code {rc})")
        path = os.path.join(self.out, f"{self.step_no}.f32")
        self.step_no += 1
        n_want = sum(len(w) for _, _, w in entries)
        if n_want == 0:
            assert not os.path.exists(path)
            return None
        flat = np.fromfile(path, dtype="<f4")
        return flat.reshape(n_want, -1)

    def close(self):
        self.proc.stdin.close()
        rc = self.proc.wait(timeout=120)
        assert rc == 0, f"trace_run exited with {rc}"

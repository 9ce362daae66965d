"""Steps allocate nothing: every activation lies in the arena that the engine built once.
Checked on the allocator's own count of allocations, across steps of every kind (a prompt
portion beside decode tokens, a long portion, single tokens launched and replayed from a
graph), in both precisions, with the logits still those of the plain implementation when the
same memory is used again and again."""

import numpy as np
import pytest
import torch

import plain_llama as P
from tiny_models import CONFIGS, model_dir

pytestmark = pytest.mark.gpu


def _allocations():
    return torch.cuda.memory_stats()["allocation.all.allocated"]


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_warmed_steps_allocate_nothing(dtype, tol, graphs):
    from kv_cache_optimization_for_llm_b200 import EngineConfig
    from kv_cache_optimization_for_llm_b200.engine.batch import StepEntry
    from kv_cache_optimization_for_llm_b200.engine.runner import ModelRunner
    mdir = model_dir("tiny_d", "float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(mdir)
    rng = np.random.default_rng(77)
    seqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (260, 90, 40)]
    refs = [P.forward(cfg, w, s) for s in seqs]
    r = ModelRunner(mdir, EngineConfig(dtype=dtype, page_size=16, num_pages=64, max_num_seqs=4,
                                       max_num_batched_tokens=256, max_model_len=320, use_cuda_graphs=graphs))

    def one_round(base):
        """A long portion; then a portion of another request beside a single token of the first;
        then single tokens of all three.  Returns the worst relative error."""
        worst = 0.0
        out = r.step([StepEntry(base, seqs[0][:200], 0, [0, 127, 128, 199])])
        worst = max(worst, np.abs(out.cpu().numpy() - refs[0][[0, 127, 128, 199]]).max() / np.abs(refs[0]).max())
        out = r.step([StepEntry(base + 1, seqs[1][:70], 0, [69]), StepEntry(base, [seqs[0][200]], 200, [0]),
                      StepEntry(base + 2, seqs[2][:30], 0, [29])])
        ref = np.stack([refs[1][69], refs[0][200], refs[2][29]])
        worst = max(worst, np.abs(out.cpu().numpy() - ref).max() / np.abs(ref).max())
        pos = [201, 70, 30]
        for _ in range(6):
            out = r.step([StepEntry(base + i, [seqs[i][pos[i]]], pos[i], [0]) for i in range(3)])
            ref = np.stack([refs[i][pos[i]] for i in range(3)])
            worst = max(worst, np.abs(out.cpu().numpy() - ref).max() / np.abs(ref).max())
            pos = [p + 1 for p in pos]
        for i in range(3):
            r.release(base + i)
        return worst

    assert one_round(0) < tol                   # warms up: kernels loaded, graphs captured, scratch made
    torch.cuda.synchronize()
    grown, before = r.arena.blocks_grown(), _allocations()
    assert one_round(10) < tol
    assert one_round(20) < tol
    torch.cuda.synchronize()
    assert _allocations() == before, "a warmed step asked the allocator for device memory"
    assert r.arena.blocks_grown() == grown == 0 and r.arena.bypassed == 0
    r.check_status()
    assert r.manager.check() == ""

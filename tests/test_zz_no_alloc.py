"""The allocation-free decode attention entry point (kvb_decode_attention_noalloc),
called through its exported C symbol the way a host that may not allocate would
call it, against the ordinary entry point that takes caller-provided scratch.

Some hosts of the kernel library cannot call cudaMalloc when they need attention
(their device memory belongs to an allocator they do not control, or an allocation's
hidden synchronisation is not allowed where they run).  For them the library keeps
16 MiB of scratch in a static device array; this test checks that the results are
the same, that a second call is not disturbed by what the first left in the array,
and that sizes beyond the array are refused with a clear message.

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2e-2}   # the tolerances of tests/test_kernels_gpu.py


def _call_noalloc(lib, c, out, nq, nkv, d, scale, window, kb, nb, dtype_code, status):
    fn = lib.kvb_decode_attention_noalloc
    fn.restype = c_int
    R = c["ctx_len"].numel()
    return fn(c_void_p(c["qkv"].data_ptr()), c_int(c["qkv"].stride(0)), c_void_p(c["kp"].data_ptr()),
              c_void_p(c["vp"].data_ptr()), c_void_p(c["table"].data_ptr()), c_int(c["table"].shape[1]),
              c_int(c["kp"].shape[2]), c_int(c["kp"].shape[0]), c_void_p(c["q_start"].data_ptr()),
              c_void_p(c["ctx_len"].data_ptr()), c_void_p(out.data_ptr()), c_int(R), c_int(nq), c_int(nkv),
              c_int(d), c_float(scale), c_int(window or 0), c_int(kb), c_int(nb), c_int(dtype_code),
              c_void_p(status.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_noalloc_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    from test_kernels_gpu import DT, _attention_case, as64, status

    lib = ops.lib("attention")
    nq, nkv, d, max_pos = 8, 2, 64, 2048
    scale = 1 / math.sqrt(d)
    kb, nb = ops.decode_key_blocks(max_pos)
    # two different batches, the second shorter: whatever the first call left in the
    # scratch beyond the second call's needs must not matter
    cases = [([700, 1, 129, 1300, 64], 11), ([200, 513, 2], 12)]
    for ctxs, seed in cases:
        c = _attention_case(dtype, nq, nkv, d, ctxs=ctxs, q_lens=[1] * len(ctxs), page_size=16, window=None,
                            seed=seed)
        st = status()
        want = ops.decode_attention(c["qkv"], c["kp"], c["vp"], c["table"], c["q_start"], c["ctx_len"], nq, nkv,
                                    d, scale, None, max_pos, st)
        got = torch.full_like(want, float("nan"))
        rc = _call_noalloc(lib, c, got, nq, nkv, d, scale, None, kb, nb, ops.dtype_code(DT[dtype]), st)
        assert rc == 0, ctypes.c_char_p(lib.kvb_decode_attention_noalloc_error(c_int(rc)))
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        ref = c["ref"]
        scale_ref = np.abs(ref).max()
        assert np.abs(as64(got) - as64(want)).max() / scale_ref < TOL[dtype]
        assert np.abs(as64(got) - ref).max() / scale_ref < TOL[dtype]


def test_noalloc_entry_point_refuses_sizes_beyond_its_scratch():
    from kv_cache_optimization_for_llm_b200 import ops
    from test_kernels_gpu import DT, _attention_case, status

    lib = ops.lib("attention")
    needed = lib.kvb_decode_attention_noalloc_scratch_needed
    needed.restype = ctypes.c_ulonglong
    err = lib.kvb_decode_attention_noalloc_error
    err.restype = ctypes.c_char_p
    nq, nkv, d = 32, 8, 128
    c = _attention_case("bfloat16", nq, nkv, d, ctxs=[5, 9], q_lens=[1, 1], page_size=16, window=None, seed=3)
    # 2 requests * 32 heads * 512 key blocks * 130 floats > 4 Mi floats
    kb, nb = 128, 512
    assert needed(c_int(2), c_int(nq), c_int(nb), c_int(d)) == 2 * nq * nb * (d + 2) > 4 * 1024 * 1024
    out = torch.full((2, nq * d), 3.0, dtype=torch.bfloat16, device="cuda")
    st = status()
    rc = _call_noalloc(lib, c, out, nq, nkv, d, 0.1, None, kb, nb, ops.dtype_code(DT["bfloat16"]), st)
    assert rc == -4
    assert b"4 Mi floats" in err(c_int(rc))
    torch.cuda.synchronize()
    assert bool((out == 3.0).all()), "a refused call must not touch the output"
    # the same sizes with few enough key blocks are served
    rc = _call_noalloc(lib, c, out, nq, nkv, d, 1 / math.sqrt(d), None, kb, 64, ops.dtype_code(DT["bfloat16"]), st)
    assert rc == 0
    torch.cuda.synchronize()
    assert np.abs(out.float().cpu().numpy() - c["ref"]).max() / np.abs(c["ref"]).max() < TOL["bfloat16"]

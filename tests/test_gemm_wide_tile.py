"""The choice of tiles of the product kernel for steps of many rows (host code of
gemm_bf16_wide.cu; needs no GPU, only the built library): which form a problem gets
when the caller leaves the choice to the kernel."""

import ctypes
from ctypes import c_int

import pytest


def _tile(M, N, epilogue):
    from kv_cache_optimization_for_llm_b200 import ops
    rows, cols, pair = c_int(0), c_int(0), c_int(0)
    rc = ops.lib("gemm_bf16_wide").kvb_gemm_wide_tile(c_int(M), c_int(N), c_int(epilogue), ctypes.byref(rows),
                                                      ctypes.byref(cols), ctypes.byref(pair))
    assert rc == 0
    return rows.value, cols.value, pair.value


@pytest.mark.parametrize("N", [3072, 2048, 16384])
def test_large_problems_go_to_pairs_of_sms(N):
    assert _tile(2048, N, 0) == (256, 256, 1)
    assert _tile(2048, 16384, 1) == (256, 256, 1)


def test_every_choice_is_a_form_the_kernel_has():
    forms = {(128, 64, 0), (128, 128, 0), (128, 256, 0), (256, 256, 0), (256, 256, 1)}
    for M in (1, 100, 128, 129, 300, 512, 1000, 2048, 5000):
        for N in (8, 64, 200, 1000, 2048, 3072, 128256):
            assert _tile(M, N, 0) in forms
            if N % 128 == 0:
                assert _tile(M, N, 1) in forms - {(128, 64, 0)}       # gate and up share a tile of 128 features
            assert _tile(M, N, 2) in {(128, 256, 0), (256, 256, 1)}   # the forms with the add-into-residual epilogue

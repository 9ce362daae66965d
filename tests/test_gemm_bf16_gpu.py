"""The tcgen05 matrix-product kernels against a float64 product of the same bfloat16
values, at sizes with ragged edges (N no multiple of 128, K no multiple of 64), with
and without K splits, both output types."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(1, 128, 64), (8, 256, 128), (5, 200, 72), (16, 128, 8), (3, 1000, 192), (64, 2048, 2048), (8, 3072, 2048),
          (8, 2048, 8192), (33, 16384, 2048), (200, 512, 256), (256, 384, 1024), (1, 2048, 8192), (17, 777 * 8, 520),
          (2, 128256, 2048)]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_skinny_matches_float64(M, N, K, out_dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_skinny(x, w, out_dtype, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = x.double() @ w.double().t()
    err = (out.double() - ref).abs().max().item()
    scale = ref.abs().max().item()
    # float32 accumulation of K products; bfloat16 output adds one rounding of 2^-9
    tol = (2e-5 if out_dtype == torch.float32 else 5e-3) * scale
    assert err < tol, (err, scale)
    # twice in a row: the split counters were left at zero, the result is bit-identical
    out2 = ops.gemm_skinny(x, w, out_dtype, st)
    assert torch.equal(out, out2)


def test_gemm_skinny_rows_do_not_depend_on_their_neighbours():
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(40, 2048, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(3072, 2048, generator=g, device="cuda") / 45).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    full = ops.gemm_skinny(x, w, torch.float32, st)
    for rows in ([0], [39], list(range(7, 12))):
        part = ops.gemm_skinny(x[rows].contiguous(), w, torch.float32, st)
        assert torch.equal(part, full[rows])
    assert int(st.item()) == 0


def test_gemm_skinny_refuses_what_it_cannot_do():
    from kv_cache_optimization_for_llm_b200 import ops
    assert ops.gemm_skinny_plan(257, 128, 64) is None      # too many rows for the skinny form
    assert ops.gemm_skinny_plan(4, 128, 100) is None       # K * 2 bytes must be a multiple of 16
    assert ops.gemm_skinny_plan(4, 128, 104) is not None


def _bf(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 8192, 2048), (16, 512, 192), (5, 192, 520), (3, 64, 2048)])
def test_swiglu_epilogue(M, I, K):
    """Product with row-interleaved gate/up weights and silu(gate)*up as its epilogue,
    against float64; and the same through the unfused pair of kernels."""
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + I + K)
    x = _bf(torch.randn(M, K, generator=g, device="cuda"))
    wg = _bf(torch.randn(I, K, generator=g, device="cuda") / K ** 0.5)
    wu = _bf(torch.randn(I, K, generator=g, device="cuda") / K ** 0.5)
    inter = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()
    gate, up = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    ref = gate / (1 + torch.exp(-gate)) * up
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    fused = ops.gemm_skinny(x, inter, torch.bfloat16, st, epilogue="swiglu")
    assert fused.shape == (M, I) and int(st.item()) == 0
    tol = 6e-3 * ref.abs().max().item()
    assert (fused.double() - ref).abs().max().item() < tol
    assert torch.equal(fused, ops.linear_swiglu(x, inter, 64))
    unfused = ops.silu_mul(ops.gemm_skinny(x, inter, torch.bfloat16, st), block=64)
    assert (unfused.double() - ref).abs().max().item() < 2 * tol   # gate and up rounded to bfloat16 in between

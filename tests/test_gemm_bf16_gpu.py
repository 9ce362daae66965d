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


@pytest.mark.parametrize("M,I,K", [(1, 128, 64), (8, 8192, 2048), (16, 512, 192), (5, 192, 520), (3, 64, 2048),
                                   (17, 8192, 2048), (64, 8192, 2048), (45, 192, 520), (64, 64, 2048)])
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
    via_dispatch = ops.linear_swiglu(x, inter, 64)            # the same kernel for few rows, the library product beyond
    assert (via_dispatch.double() - ref).abs().max().item() < 2 * tol
    if M <= min(ops.SKINNY_MAX_ROWS, ops.FUSED_EPILOGUE_MAX_ROWS):
        assert torch.equal(fused, via_dispatch)
    unfused = ops.silu_mul(ops.gemm_skinny(x, inter, torch.bfloat16, st), block=64)
    assert (unfused.double() - ref).abs().max().item() < 2 * tol   # gate and up rounded to bfloat16 in between


# ---- the residual stream folded into the products: add in the epilogue, 1/rms as a row scale

@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 2048, 2048), (8, 2048, 8192), (5, 200, 72), (16, 1000, 520),
                                   (3, 96, 1024), (17, 2048, 2048), (33, 2048, 8192), (64, 2048, 2048), (50, 200, 72),
                                   (64, 1000, 520)])
def test_residual_epilogue(M, N, K):
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = _bf(torch.randn(M, K, generator=g, device="cuda"))
    w = _bf(torch.randn(N, K, generator=g, device="cuda") / K ** 0.5)
    resid0 = torch.randn(M, N, generator=g, device="cuda") * 3
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    resid = resid0.clone()
    folded = ops.gemm_skinny_fused(x, w, st, into=resid)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and isinstance(folded, ops.Folded)
    ref = resid0.double() + x.double() @ w.double().t()
    scale = ref.abs().max().item()
    assert (resid.double() - ref).abs().max().item() < 2e-5 * scale     # float32 sum, no bfloat16 rounding between
    assert torch.equal(folded.xb, resid.to(torch.bfloat16))              # the bfloat16 copy is the new residual, rounded once
    # the partial sums cover every feature once: together they are the squared norm of the new rows
    assert folded.sumsq.shape == (M, -(-N // 128))
    total = folded.sumsq.double().sum(dim=1)
    want = (resid.double() ** 2).sum(dim=1)
    assert ((total - want).abs() / want).max().item() < 1e-5
    # each part is its own tile's sum
    t = min(N, 128)
    assert ((folded.sumsq[:, 0].double() - (resid[:, :t].double() ** 2).sum(dim=1)).abs() / want).max().item() < 1e-5
    # a row's result does not depend on the rows beside it
    if M > 1:
        r2 = resid0[M - 1:].clone()
        f2 = ops.gemm_skinny_fused(x[M - 1:].contiguous(), w, st, into=r2)
        assert torch.equal(r2, resid[M - 1:]) and torch.equal(f2.sumsq, folded.sumsq[M - 1:])
        assert torch.equal(f2.xb, folded.xb[M - 1:])


@pytest.mark.parametrize("epilogue", ["store", "swiglu"])
@pytest.mark.parametrize("M,N,K,parts,eps", [(1, 128, 64, 1, 1e-5), (8, 3072, 2048, 16, 1e-5), (8, 16384, 2048, 16, 1e-6),
                                             (5, 256, 72, 3, 1e-3), (16, 1024, 520, 5, 1e-5), (16, 16384, 2048, 16, 1e-5),
                                             (2, 384, 4096, 32, 1e-5), (7, 128, 8192, 64, 1e-5),
                                             (17, 3072, 2048, 16, 1e-5), (64, 16384, 2048, 16, 1e-5),
                                             (35, 1024, 520, 5, 1e-5), (64, 3072, 2048, 16, 1e-5), (40, 128, 64, 1, 1e-5)])
def test_row_scale(M, N, K, parts, eps, epilogue):
    """x . w^T with every row scaled by the 1/rms that follows from partial sums of squares."""
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    resid = torch.randn(M, K, generator=g, device="cuda") * torch.linspace(0.5, 4.0, M, device="cuda")[:, None]
    xb = _bf(resid)
    w = _bf(torch.randn(N, K, generator=g, device="cuda") / K ** 0.5)
    # the row's sum of squares, cut into parts in some uneven way
    total = (resid.double() ** 2).sum(dim=1)
    cut = torch.rand(M, parts, generator=g, device="cuda").double() + 0.1
    sumsq = (cut / cut.sum(dim=1, keepdim=True) * total[:, None]).float().contiguous()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    pn = ops.PendingNorm(resid, xb, sumsq, eps, torch.bfloat16)
    out = ops.gemm_skinny_fused(xb, w, st, row_scale=pn, epilogue=epilogue)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    rstd = 1.0 / torch.sqrt(total / K + eps)
    ref = (xb.double() @ w.double().t()) * rstd[:, None]
    if epilogue == "swiglu":
        ref = ref.view(M, N // 128, 2, 64)
        gate, up = ref[:, :, 0], ref[:, :, 1]
        ref = (gate * torch.sigmoid(gate) * up).reshape(M, N // 2)
    scale = ref.abs().max().item()
    assert (out.double() - ref).abs().max().item() < 5e-3 * scale      # the output's own bfloat16 rounding
    # against the separate weightless norm kernel followed by the plain product: the rows are
    # rounded to bfloat16 before the scale there and after it here
    sep = ops.gemm_skinny(pn.materialize(), w, torch.bfloat16, st, epilogue=epilogue)
    assert (out.double() - sep.double()).abs().max().item() < 1e-2 * scale
    # rows alone give the same bits
    if M > 1:
        i = 2 % M
        one = ops.gemm_skinny_fused(xb[i:i + 1].contiguous(), w, st, epilogue=epilogue,
                                    row_scale=ops.PendingNorm(resid[i:i + 1], xb[i:i + 1], sumsq[i:i + 1].contiguous(),
                                                              eps, torch.bfloat16))
        assert torch.equal(one, out[i:i + 1])


def test_weightless_norm_kernel():
    from kv_cache_optimization_for_llm_b200 import ops
    for H in (2048, 72, 1000):
        resid = torch.randn(5, H, device="cuda") * 2
        got = ops.add_rmsnorm(resid.clone(), None, None, 1e-5, torch.float32)
        want = ops.add_rmsnorm(resid.clone(), None, torch.ones(H, device="cuda"), 1e-5, torch.float32)
        assert torch.equal(got, want)


def test_a_wait_that_runs_out_reports_and_returns():
    """Every barrier wait of the tensor-core kernels has a limit; when it runs out the kernel
    records a status the host can read and returns.  Here the limit is short and the barrier
    is one that nothing completes; afterwards the device works as before."""
    from kv_cache_optimization_for_llm_b200 import ops
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.wait_selftest(2000, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 4 and "wait" in ops.STATUS_TEXT[4].lower()
    st.zero_()
    x = _bf(torch.randn(4, 256, device="cuda"))
    w = _bf(torch.randn(128, 256, device="cuda") / 16)
    out = ops.gemm_skinny(x, w, torch.float32, st)
    assert int(st.item()) == 0
    assert (out.double() - x.double() @ w.double().t()).abs().max().item() < 1e-3


def test_every_number_of_rows_up_to_64():
    """The split-K partials travel in groups of four rows to their owner blocks; the last group
    may be partly filled and, with few rows, most blocks own nothing.  Every row count from 1
    to 64, with K split eight ways: store, add-into-residual with its sums of squares, and the
    row scale."""
    from kv_cache_optimization_for_llm_b200 import ops
    N, K = 256, 1024                       # two tiles of 128 features, eight blocks along K
    assert ops.gemm_skinny_plan(8, N, K)[0] == 8
    g = torch.Generator(device="cuda").manual_seed(0)
    w = _bf(torch.randn(N, K, generator=g, device="cuda") / K ** 0.5)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    for M in range(1, 65):
        x = _bf(torch.randn(M, K, generator=g, device="cuda"))
        ref = x.double() @ w.double().t()
        scale = ref.abs().max().item()
        out = ops.gemm_skinny(x, w, torch.float32, st)
        assert (out.double() - ref).abs().max().item() < 2e-5 * scale, M
        resid0 = torch.randn(M, N, generator=g, device="cuda")
        resid = resid0.clone()
        folded = ops.gemm_skinny_fused(x, w, st, into=resid)
        assert (resid.double() - (resid0.double() + ref)).abs().max().item() < 2e-5 * (scale + 4), M
        want = (resid.double() ** 2).sum(dim=1)
        assert ((folded.sumsq.double().sum(dim=1) - want).abs() / want).max().item() < 1e-5, M
        sumsq = (x.float() ** 2).sum(dim=1, keepdim=True).contiguous()
        pn = ops.PendingNorm(x.float(), x, sumsq, 1e-5, torch.bfloat16)
        scaled = ops.gemm_skinny_fused(x, w, st, row_scale=pn)
        rstd = 1.0 / torch.sqrt(sumsq.double() / K + 1e-5)
        assert (scaled.double() - ref * rstd).abs().max().item() < 5e-3 * (ref * rstd).abs().max().item(), M
    assert int(st.item()) == 0


# ------------------------------------------------------------------ the kernel for steps of many rows

WIDE_SHAPES = [(128, 256, 64), (130, 264, 72), (1, 8, 8), (300, 1000, 200), (2048, 3072, 2048), (517, 2048, 8192),
               (1000, 777 * 8, 520), (129, 16384, 256)]


@pytest.mark.parametrize("tile", [(0, 0), (128, 64), (128, 128), (128, 256), (256, 256), (256, 256, 1)])
@pytest.mark.parametrize("M,N,K", WIDE_SHAPES)
def test_gemm_wide_matches_float64(M, N, K, tile):
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_wide(x, w, st, tile=tile)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = x.double() @ w.double().t()
    err = (out.double() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err < 5e-3 * scale, (err, scale)     # float32 accumulation, one bfloat16 rounding of 2^-9
    assert torch.equal(out, ops.gemm_wide(x, w, st, tile=tile))


def test_gemm_wide_finds_one_large_product_anywhere():
    """One element of x and one of w made large: exactly one output stands out, wherever the
    pair lies (a tile's last row, the last feature, the last element of K)."""
    from kv_cache_optimization_for_llm_b200 import ops
    M, N, K = 391, 1544, 1096
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    for (m, n, k) in [(0, 0, 0), (127, 255, 63), (128, 256, 64), (390, 1543, 1095), (255, 1300, 1087)]:
        x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
        w = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
        x[m, k] = 3.0
        w[n, k] = 5.0
        out = ops.gemm_wide(x, w, st).float()
        assert torch.equal(out, ops.gemm_wide(x, w, st, tile=(256, 256)).float())
        assert torch.equal(out, ops.gemm_wide(x, w, st, tile=(256, 256, 1)).float())
        assert out[m, n].item() == 15.0
        out[m, n] = 0
        assert out.abs().max().item() == 0.0
    assert int(st.item()) == 0


@pytest.mark.parametrize("tile", [(0, 0), (128, 128), (128, 256), (256, 256), (256, 256, 1)])
@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (333, 704, 200), (2048, 8192, 2048)])
def test_gemm_wide_swiglu_epilogue(M, I, K, tile):
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    gate = (torch.randn(I, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    up = (torch.randn(I, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    # rows in blocks of 128: 64 gate features, then the 64 up features of the same indices
    gu = torch.stack([gate.view(I // 64, 64, K), up.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_wide(x, gu, st, epilogue="swiglu", tile=tile)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and out.shape == (M, I)
    gd, ud = x.double() @ gate.double().t(), x.double() @ up.double().t()
    ref = gd / (1 + torch.exp(-gd)) * ud
    err = (out.double() - ref).abs().max().item()
    assert err < 5e-3 * ref.abs().max().item() + 1e-6


def test_gemm_wide_rows_do_not_depend_on_their_neighbours():
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(400, 2048, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(3072, 2048, generator=g, device="cuda") / 45).to(torch.bfloat16)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    full = ops.gemm_wide(x, w, st)
    for rows in (slice(0, 1), slice(399, 400), slice(100, 329)):
        assert torch.equal(ops.gemm_wide(x[rows].contiguous(), w, st), full[rows])
    assert int(st.item()) == 0


def test_gemm_wide_refuses_what_it_cannot_do():
    from kv_cache_optimization_for_llm_b200 import ops
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.zeros(128, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError):
        ops.gemm_wide(x, torch.zeros(64, 100, dtype=torch.bfloat16, device="cuda"), st)     # K no multiple of 8
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError):
        ops.gemm_wide(x, torch.zeros(60, 64, dtype=torch.bfloat16, device="cuda"), st)      # N no multiple of 8
    with pytest.raises(ops.KernelError):
        ops.gemm_wide(x, torch.zeros(192, 64, dtype=torch.bfloat16, device="cuda"), st, epilogue="swiglu")


@pytest.mark.parametrize("tile", [(0, 0), (128, 256), (256, 256), (256, 256, 1)])
@pytest.mark.parametrize("M,N,K,parts", [(200, 256, 192, 1), (517, 1024, 520, 5), (2048, 3072, 2048, 8)])
def test_gemm_wide_row_scale(M, N, K, parts, tile):
    """The product over bare rows, every row scaled by the 1/rms that follows from partial sums of
    squares (the norm in front of it, not carried out), plain and with the SiLU * up epilogue."""
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    sumsq = (torch.rand(M, parts, generator=g, device="cuda") * K / parts * 4).contiguous()
    eps = 1e-5
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    pending = ops.PendingNorm(None, x, sumsq, eps, torch.bfloat16)
    rstd = 1.0 / torch.sqrt(sumsq.double().sum(1) / K + eps)
    ref = (x.double() @ w.double().t()) * rstd[:, None]
    out = ops.gemm_wide(x, w, st, tile=tile, row_scale=pending)
    assert (out.double() - ref).abs().max().item() < 5e-3 * ref.abs().max().item()
    I = N // 2
    gd = torch.cat([ref[:, i:i + 64] for i in range(0, N, 128)], dim=1)
    ud = torch.cat([ref[:, i + 64:i + 128] for i in range(0, N, 128)], dim=1)
    ref2 = gd / (1 + torch.exp(-gd)) * ud
    out2 = ops.gemm_wide(x, w, st, epilogue="swiglu", tile=tile, row_scale=pending)
    assert out2.shape == (M, I)
    assert (out2.double() - ref2).abs().max().item() < 5e-3 * ref2.abs().max().item() + 1e-6
    assert int(st.item()) == 0


@pytest.mark.parametrize("tile", [(0, 0), (128, 256), (256, 256, 1)])
@pytest.mark.parametrize("M,N,K", [(200, 192, 512), (391, 1000, 264), (2048, 2048, 8192)])
def test_gemm_wide_adds_into_the_residual(M, N, K, tile):
    """resid += x . w^T in float32 and in place; the new rows in bfloat16; partial sums of their
    squares per 256 features that add up to the rows' sums of squares."""
    from kv_cache_optimization_for_llm_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M * 3 + N + K)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    resid = torch.randn(M, N, generator=g, device="cuda")
    ref = resid.double() + x.double() @ w.double().t()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    folded = ops.gemm_wide(x, w, st, tile=tile, into=resid)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    scale = ref.abs().max().item()
    assert (resid.double() - ref).abs().max().item() < 2e-5 * scale
    assert torch.equal(folded.xb, resid.to(torch.bfloat16))
    assert folded.sumsq.shape == (M, -(-N // 256))
    ss = (resid.double() ** 2).sum(1)
    assert ((folded.sumsq.double().sum(1) - ss).abs() / ss).max().item() < 1e-5
    for t in range(folded.sumsq.shape[1]):
        part = (resid[:, 256 * t:256 * (t + 1)].double() ** 2).sum(1)
        assert ((folded.sumsq[:, t].double() - part).abs() / (part + 1e-9)).max().item() < 1e-5

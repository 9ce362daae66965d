"""Each kernel alone against the plain implementation, at sizes other than the tiny
models': widths and vocabularies that are no power of two, head sizes 16..256,
groups 1..8, page edges, a window's edge, and inputs made so that a single far key
decides the result."""

import math

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def dev(x, dtype=None):
    t = torch.as_tensor(np.asarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def as64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def rel_err(got, ref):
    return np.abs(as64(got) - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 48), (5, 1000), (3, 2048), (2, 13000)])
def test_add_rmsnorm(dtype, T, H):
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(T * H)
    resid = rng.normal(size=(T, H)) * 3
    delta = as64(dev(rng.normal(size=(T, H)), DT[dtype]))
    w = 1 + 0.1 * rng.normal(size=H)
    w = as64(dev(w, torch.float32))
    r0 = as64(dev(resid, torch.float32))
    rd = dev(resid, torch.float32)
    out = ops.add_rmsnorm(rd, dev(delta, DT[dtype]), dev(w, torch.float32), 1e-5, DT[dtype])
    ref_sum = r0 + delta
    assert np.abs(as64(rd) - ref_sum).max() < 1e-6 * np.abs(ref_sum).max()        # the residual sum is float32
    assert rel_err(out, P.rms_norm(ref_sum, w, 1e-5)) < TOL[dtype]
    # no delta; and selected rows only, residual untouched
    rd2 = dev(resid, torch.float32)
    out = ops.add_rmsnorm(rd2, None, dev(w, torch.float32), 1e-5, DT[dtype])
    assert rel_err(out, P.rms_norm(r0, w, 1e-5)) < TOL[dtype] and np.array_equal(as64(rd2), r0)
    rows = [T - 1, 0]
    out = ops.add_rmsnorm(rd2, dev(delta, DT[dtype]), dev(w, torch.float32), 1e-5, DT[dtype],
                          rows=dev(rows, torch.int32))
    assert rel_err(out, P.rms_norm(ref_sum[rows], w, 1e-5)) < TOL[dtype] and np.array_equal(as64(rd2), r0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul_and_embedding(dtype):
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(0)
    gu = as64(dev(rng.normal(size=(7, 2 * 333)) * 4, DT[dtype]))
    out = ops.silu_mul(dev(gu, DT[dtype]))
    g, u = gu[:, :333], gu[:, 333:]
    assert rel_err(out, g / (1 + np.exp(-g)) * u) < TOL[dtype]
    # rows that hold gate and up in alternating blocks, at widths that take the 4-wide, the 8-wide
    # (bfloat16) and the one-by-one form
    for inter, block in ((384, 64), (200, 8), (100, 4), (99, 3)):
        gu = as64(dev(rng.normal(size=(5, 2 * inter)) * 4, DT[dtype]))
        out = ops.silu_mul(dev(gu, DT[dtype]), block=block)
        v = gu.reshape(5, inter // block, 2, block)
        g, u = v[:, :, 0].reshape(5, inter), v[:, :, 1].reshape(5, inter)
        assert rel_err(out, g / (1 + np.exp(-g)) * u) < TOL[dtype], (inter, block)
    table = as64(dev(rng.normal(size=(777, 100)), DT[dtype]))
    ids = [0, 776, 5, 5, 300]
    st = status()
    out = ops.embed_gather(dev(table, DT[dtype]), dev(ids, torch.int32), st)
    assert out.dtype == torch.float32 and np.array_equal(as64(out), table[ids]) and int(st.item()) == 0
    ops.embed_gather(dev(table, DT[dtype]), dev([3, 777], torch.int32), st)
    assert int(st.item()) == 3      # a token outside the table is reported, not read


@pytest.mark.parametrize("M,N,K", [(1, 1000, 192), (5, 77, 33), (70, 130, 517), (64, 64, 16), (3, 128256 // 8, 100)])
def test_sgemm_is_true_float32_and_row_independent(M, N, K):
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(M + N + K)
    a = rng.normal(size=(M, K)).astype(np.float32)
    w = rng.normal(size=(N, K)).astype(np.float32)
    out = ops.linear(dev(a), dev(w))
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    # float32 FMA chains of length K: error ~ K * 2^-24 relative to the sum of magnitudes
    bound = (np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64).T) * K * 2.0 ** -24
    assert (np.abs(as64(out) - ref) <= bound + 1e-30).all()
    # a tf32 product would miss by ~2^-11 relative: make sure we are far below that
    assert np.abs(as64(out) - ref).max() < 1e-5 * np.abs(ref).max()
    # a row's result does not depend on the rows beside it: bit for bit
    one = ops.linear(dev(a[M - 1:M]), dev(w))
    assert torch.equal(one[0], out[M - 1])


def _paged(k, v, page_size, num_pages, rng, dtype):
    """Scatters one sequence's keys/values [ctx, nkv, d] into randomly chosen pages.
    Returns (k_pages, v_pages, table)."""
    ctx, nkv, d = k.shape
    n = -(-ctx // page_size)
    table = rng.permutation(num_pages)[:n]
    kp = np.zeros((num_pages, nkv, page_size, d))
    vp = np.zeros_like(kp)
    kp[:] = 7.0   # poison: an unmapped or stale slot read by mistake shows up
    vp[:] = -9.0
    for j in range(ctx):
        kp[table[j // page_size], :, j % page_size] = k[j]
        vp[table[j // page_size], :, j % page_size] = v[j]
    return kp, vp, table


def _attention_case(dtype, nq, nkv, d, ctxs, q_lens, page_size, window, seed, spike=None):
    """Several requests, each with ``q_len`` newest tokens as queries over ``ctx`` cached
    keys.  Returns what the kernels need and the plain result per token."""
    rng = np.random.default_rng(seed)
    R = len(ctxs)
    max_pages = max(-(-c // page_size) for c in ctxs) + 2
    num_pages = sum(-(-c // page_size) for c in ctxs) + 3
    kp = np.full((num_pages, nkv, page_size, d), 7.0)
    vp = np.full((num_pages, nkv, page_size, d), -9.0)
    free = list(rng.permutation(num_pages))
    tables = np.full((R, max_pages), -1, dtype=np.int32)
    qkv_rows, positions, token_req, refs, q_start, ctx_len = [], [], [], [], [0], []
    for r, (ctx, ql) in enumerate(zip(ctxs, q_lens)):
        k = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))
        v = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))
        q = as64(dev(rng.normal(size=(ctx, nq, d)), DT[dtype]))
        if spike is not None:
            # one far key matches the last query exactly and strongly: if it is skipped
            # or misplaced the output is visibly wrong
            j = spike if spike < ctx else 0
            k[:, :, 0] = 0.0          # no other key answers along dim 0
            k[j] = 0.0
            k[j, :, 0] = 1.0
            q[ctx - 1] = 0.0
            q[ctx - 1, :, 0] = 12.0 * math.sqrt(d)
            k[j], q[ctx - 1] = as64(dev(k[j], DT[dtype])), as64(dev(q[ctx - 1], DT[dtype]))
        for j in range(ctx):
            lp = j // page_size
            if tables[r, lp] < 0:
                tables[r, lp] = free.pop()
            kp[tables[r, lp], :, j % page_size] = k[j]
            vp[tables[r, lp], :, j % page_size] = v[j]
        full = P.attention(q, k, v, window=window)
        for i in range(ctx - ql, ctx):
            row = np.concatenate([q[i].reshape(-1), np.zeros(2 * nkv * d)])
            qkv_rows.append(row)
            positions.append(i)
            token_req.append(r)
            refs.append(full[i].reshape(-1))
        q_start.append(len(qkv_rows))
        ctx_len.append(ctx)
    return dict(qkv=dev(np.array(qkv_rows), DT[dtype]), kp=dev(kp, DT[dtype]), vp=dev(vp, DT[dtype]),
                table=dev(tables, torch.int32), positions=dev(positions, torch.int32),
                token_req=dev(token_req, torch.int32), q_start=dev(q_start, torch.int32),
                ctx_len=dev(ctx_len, torch.int32), ref=np.array(refs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,page_size,window", [
    (4, 2, 16, 4, None), (6, 1, 32, 16, None), (5, 5, 48, 16, None), (8, 2, 64, 16, None),
    (3, 1, 128, 32, None), (2, 2, 256, 8, None), (4, 2, 64, 16, 37), (6, 3, 32, 4, 5),
])
def test_generic_attention_mixed_runs(dtype, nq, nkv, d, page_size, window):
    from kv_cache_optimization_for_llm_b200 import ops
    c = _attention_case(dtype, nq, nkv, d, ctxs=[1, 33, 130, 64, 257], q_lens=[1, 33, 2, 1, 40],
                        page_size=page_size, window=window, seed=d + nq)
    st = status()
    out = ops.paged_attention_generic(c["qkv"], c["kp"], c["vp"], c["table"], c["positions"], c["token_req"],
                                      nq, nkv, d, 1 / math.sqrt(d), window, st)
    assert int(st.item()) == 0
    assert rel_err(out, c["ref"]) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,page_size,window,max_pos", [
    (8, 2, 64, 16, None, 4096), (32, 8, 64, 16, None, 1024), (6, 1, 32, 16, None, 1024), (24, 8, 128, 16, None, 20000),
    (8, 8, 128, 32, None, 4096), (16, 2, 64, 8, None, 4096), (8, 2, 64, 16, 100, 4096), (4, 4, 32, 4, 129, 2048),
])
def test_decode_attention_split_kernel(dtype, nq, nkv, d, page_size, window, max_pos):
    from kv_cache_optimization_for_llm_b200 import ops
    ctxs = [1, 128, 129, 640, 300, 2, 1000]
    c = _attention_case(dtype, nq, nkv, d, ctxs=ctxs, q_lens=[1] * len(ctxs), page_size=page_size,
                        window=window, seed=nq * d)
    st = status()
    assert ops.decode_attention_supported(d, nq // nkv)
    out = ops.decode_attention(c["qkv"], c["kp"], c["vp"], c["table"], c["q_start"], c["ctx_len"], nq, nkv, d,
                               1 / math.sqrt(d), window, max_pos, st)
    assert int(st.item()) == 0
    assert rel_err(out, c["ref"]) < TOL[dtype]
    # a context beyond what the scratch was sized for is reported, not computed wrongly
    ops.decode_attention(c["qkv"], c["kp"], c["vp"], c["table"], c["q_start"], c["ctx_len"], nq, nkv, d,
                         1 / math.sqrt(d), window, 512, st)
    assert int(st.item()) == 2


@pytest.mark.parametrize("kernel", ["generic", "decode"])
@pytest.mark.parametrize("spike", [0, 127, 128, 511, 777])
def test_a_far_key_among_hundreds_is_found(kernel, spike):
    """The last query matches exactly one key, far back: the output must be that key's
    value.  A kernel that drops a key at a page edge, a warp's chunk edge or a key
    block's edge gives something else entirely."""
    from kv_cache_optimization_for_llm_b200 import ops
    nq, nkv, d = 8, 2, 64
    c = _attention_case("bfloat16", nq, nkv, d, ctxs=[900], q_lens=[1], page_size=16, window=None, seed=spike,
                        spike=spike)
    st = status()
    if kernel == "generic":
        out = ops.paged_attention_generic(c["qkv"], c["kp"], c["vp"], c["table"], c["positions"], c["token_req"],
                                          nq, nkv, d, 1 / math.sqrt(d), None, st)
    else:
        out = ops.decode_attention(c["qkv"], c["kp"], c["vp"], c["table"], c["q_start"], c["ctx_len"], nq, nkv, d,
                                   1 / math.sqrt(d), None, 4096, st)
    assert rel_err(out, c["ref"]) < TOL["bfloat16"]
    # and the reference itself is dominated by that key (weight > 0.99)
    page, slot = int(c["table"][0, spike // 16]), spike % 16
    v_spike = as64(c["vp"][page, :, slot])                 # [nkv, d]
    want = np.repeat(v_spike, nq // nkv, axis=0).reshape(-1)
    assert np.abs(c["ref"][0] - want).max() < 0.05


def test_unmapped_page_is_reported_not_read():
    from kv_cache_optimization_for_llm_b200 import ops
    c = _attention_case("float32", 4, 2, 16, ctxs=[40], q_lens=[1], page_size=4, window=None, seed=1)
    table = c["table"].clone()
    table[0, 3] = -1
    st = status()
    ops.paged_attention_generic(c["qkv"], c["kp"], c["vp"], table, c["positions"], c["token_req"], 4, 2, 16, 0.25,
                                None, st)
    assert int(st.item()) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,rot,page_size", [(4, 2, 16, 16, 4), (6, 1, 32, 32, 16), (5, 5, 48, 48, 16),
                                                    (8, 2, 64, 32, 8), (2, 1, 128, 128, 16)])
def test_rope_and_cache_write(dtype, nq, nkv, d, rot, page_size):
    from kv_cache_optimization_for_llm_b200 import ops
    from kv_cache_optimization_for_llm_b200.parts.position import rope_inv_freq
    rng = np.random.default_rng(d)
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    inv = rope_inv_freq(rot, 500000.0, scaling).numpy()
    assert np.allclose(inv, P.rope_inv_freq(rot, 500000.0, scaling), rtol=1e-12)
    max_pos = 300
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    cos_t, sin_t = dev(np.cos(ang), torch.float32), dev(np.sin(ang), torch.float32)
    # two requests: tokens at positions 250..255 of request 0 and 0..2 of request 1
    positions = [250, 251, 252, 253, 254, 255, 0, 1, 2]
    token_req = [0] * 6 + [1] * 3
    T = len(positions)
    qkv = as64(dev(rng.normal(size=(T, (nq + 2 * nkv) * d)), DT[dtype]))
    num_pages, max_pages = 40, 256 // page_size + 1
    table = np.full((2, max_pages), -1, dtype=np.int32)
    pages = rng.permutation(num_pages)
    table[0, 250 // page_size: 255 // page_size + 1] = pages[:255 // page_size - 250 // page_size + 1]
    table[1, 0] = pages[10]
    kp = torch.full((num_pages, nkv, page_size, d), 5.0, dtype=DT[dtype], device="cuda")
    vp = torch.full((num_pages, nkv, page_size, d), 5.0, dtype=DT[dtype], device="cuda")
    dq = dev(qkv, DT[dtype])
    st = status()
    ops.rope_kv_write(dq, dev(positions, torch.int32), dev(token_req, torch.int32), cos_t, sin_t, kp, vp,
                      dev(table, torch.int32), page_size, nq, nkv, d, rot, st)
    assert int(st.item()) == 0
    q = qkv[:, :nq * d].reshape(T, nq, d)
    k = qkv[:, nq * d:(nq + nkv) * d].reshape(T, nkv, d)
    v = qkv[:, (nq + nkv) * d:].reshape(T, nkv, d)
    c, s = np.cos(ang[positions]), np.sin(ang[positions])
    def rotate(x):
        out = x.copy()
        out[..., :rot] = P.apply_rope(x[..., :rot], c, s)
        return out
    got = as64(dq)
    assert np.abs(got[:, :nq * d].reshape(T, nq, d) - rotate(q)).max() < TOL[dtype] * 4
    assert np.array_equal(got[:, nq * d:], qkv[:, nq * d:])          # k and v stay as they were in the row
    kr = rotate(k)
    written = np.zeros((num_pages, page_size), dtype=bool)
    for t, (p, r) in enumerate(zip(positions, token_req)):
        page, slot = table[r, p // page_size], p % page_size
        written[page, slot] = True
        assert np.abs(as64(kp[page, :, slot]) - kr[t]).max() < TOL[dtype] * 4
        assert np.array_equal(as64(vp[page, :, slot]), v[t])
    # nothing else in the pool was touched
    untouched = ~written
    assert (as64(kp).transpose(0, 2, 1, 3)[untouched] == 5.0).all() and (as64(vp).transpose(0, 2, 1, 3)[untouched] == 5.0).all()
    # a position whose page is not mapped is reported and skipped
    ops.rope_kv_write(dev(qkv, DT[dtype]), dev([100] * T, torch.int32), dev(token_req, torch.int32), cos_t, sin_t,
                      kp, vp, dev(table, torch.int32), page_size, nq, nkv, d, rot, st)
    assert int(st.item()) == 1


@pytest.mark.parametrize("V", [100, 1000, 128256, 50257])
def test_sampling_kernel(V):
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(V)
    R = 6
    logits = rng.normal(0, 2.0, size=(R, V)).astype(np.float32)
    logits[:, rng.choice(V, 5, replace=False)] += 6.0
    logits[1, [V - 1, 17]] = 50.0          # a tie: the lower index wins
    logits[2, 0] = 60.0
    dl = dev(logits)
    ids = ops.sample(dl, None, None, None, None, None, None, None).cpu().numpy()
    assert ids.tolist() == [P.argmax_lowest(logits[r].astype(np.float64)) for r in range(R)]
    assert ids[1] == 17 and ids[2] == 0
    temps = np.array([0.7, 1.0, 1.5, 0.0, 0.3, 2.0], dtype=np.float32)
    seeds = np.array([1, 2, 3, 4, 2 ** 32 - 1, 0], dtype=np.uint32)
    keys = np.array([0, 7, 8 * 31 + 3, 5, 2 ** 31, 9], dtype=np.uint32)
    for pos in (0, 1, 513, 70000):
        poss = np.full(R, pos, dtype=np.uint32)
        got = ops.sample(dl, dev(temps), dev(seeds.view(np.int32)), dev(keys.view(np.int32)),
                         dev(poss.view(np.int32)), None, None, None).cpu().numpy()
        for r in range(R):
            want = P.sample(logits[r].astype(np.float64), float(temps[r]), int(seeds[r]), int(keys[r]), pos)
            assert got[r] == want, (r, pos)
    # repetition penalty through the slots' records
    mask = torch.zeros((4, V), dtype=torch.uint8, device="cuda")
    seen = {0: [int(ids[0]), 3], 2: [int(ids[2])]}
    slots = np.array([0, 1, 2, 3, 1, 3], dtype=np.int32)
    for slot, toks in seen.items():
        ops.reset_mask(mask, slot, dev(toks, torch.int32))
    pen = np.array([1.15, 1.0, 2.0, 1.15, 1.0, 1.0], dtype=np.float32)
    got = ops.sample(dl, None, None, None, None, dev(pen), mask, dev(slots)).cpu().numpy()
    for r in range(R):
        want = P.sample(logits[r].astype(np.float64), 0.0, 0, 0, 0, seen=seen.get(int(slots[r]), []), penalty=float(pen[r]))
        assert got[r] == want, r
    assert mask[0, got[0]] == 1 and mask[2, got[2]] == 1 and int(mask[1].sum()) == 0   # new tokens are recorded


class _FakeBatch:
    """What ops.flash_attention reads of a step: rows of the runs and their positions."""
    def __init__(self, c):
        self.positions, self.token_ids, self.status = c["positions"], c["positions"], status()
        self.num_reqs = c["ctx_len"].numel()
        self.host = {"q_start": c["q_start"].cpu().numpy()}


@pytest.mark.parametrize("nq,nkv,d,page_size,window", [
    (8, 2, 64, 16, None), (32, 8, 64, 16, None), (6, 2, 64, 8, None), (5, 5, 64, 4, None), (24, 8, 128, 16, None),
    (8, 1, 128, 32, None), (16, 1, 64, 64, None), (8, 2, 64, 16, 100), (4, 4, 128, 16, 33), (3, 1, 64, 16, 64),
])
def test_flash_attention_mixed_runs(nq, nkv, d, page_size, window):
    """Tensor-core kernel: whole prompts, continued prompts, a two-token portion and
    single tokens in one step; runs longer than a tile, contexts across many key tiles."""
    from kv_cache_optimization_for_llm_b200 import ops
    assert ops.flash_attention_supported(d, nq // nkv, page_size)
    c = _attention_case("bfloat16", nq, nkv, d, ctxs=[1, 70, 130, 64, 400, 257, 2], q_lens=[1, 70, 2, 1, 150, 40, 2],
                        page_size=page_size, window=window, seed=d + nq + page_size)
    for wide in (False, True) + ((2,) if d == 64 else ()) + ((3,) if page_size >= 8 else ()):   # 64 and 128 query rows per block (mma.sync), 128 on tcgen05 (two forms; the one with roles also at head size 128)
        fb = _FakeBatch(c)
        out = ops.flash_attention(c["qkv"], c["kp"], c["vp"], c["table"], fb, nq, nkv, d, 1 / math.sqrt(d), window,
                                  wide=wide)
        assert int(fb.status.item()) == 0
        assert rel_err(out, c["ref"]) < TOL["bfloat16"], wide


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("spike", [0, 63, 64, 511, 777])
def test_flash_attention_finds_a_far_key(spike, d):
    from kv_cache_optimization_for_llm_b200 import ops
    nq, nkv = (8, 2) if d == 64 else (6, 2)
    c = _attention_case("bfloat16", nq, nkv, d, ctxs=[900], q_lens=[37], page_size=16, window=None, seed=spike,
                        spike=spike)
    for wide in (None, 2, 3) if d == 64 else (None, True, 3):
        fb = _FakeBatch(c)
        out = ops.flash_attention(c["qkv"], c["kp"], c["vp"], c["table"], fb, nq, nkv, d, 1 / math.sqrt(d), None,
                                  wide=wide)
        assert int(fb.status.item()) == 0
        assert rel_err(out, c["ref"]) < TOL["bfloat16"], wide
        page, slot = int(c["table"][0, spike // 16]), spike % 16
        want = np.repeat(as64(c["vp"][page, :, slot]), nq // nkv, axis=0).reshape(-1)
        assert np.abs(as64(out)[-1] - want).max() < 0.08, wide      # the last query sees that key's value


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,rot,page_size,window,write", [
    (8, 2, 64, 64, 16, None, True), (32, 8, 64, 64, 16, None, True), (6, 1, 32, 32, 16, None, True),
    (24, 8, 128, 128, 16, None, True), (8, 2, 64, 32, 8, None, True), (8, 2, 64, 64, 16, 100, True),
    (4, 4, 32, 32, 4, 129, True), (8, 2, 64, 64, 16, None, False)])
def test_fused_decode_attention(dtype, nq, nkv, d, rot, page_size, window, write):
    """One launch does rotary encoding, the cache write, split attention and the merge:
    against rotate-then-attend in float64.  The cache holds everything but the newest
    key/value of each request, which the kernel has to put there itself."""
    from kv_cache_optimization_for_llm_b200 import ops
    rng = np.random.default_rng(nq * d + rot)
    ctxs = [1, 128, 129, 640, 300, 2, 1000]
    R = len(ctxs)
    max_pos = 1024
    inv = P.rope_inv_freq(rot, 10000.0)
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    cos_t, sin_t = dev(np.cos(ang), torch.float32), dev(np.sin(ang), torch.float32)
    max_pages = max(-(-c // page_size) for c in ctxs) + 1
    num_pages = sum(-(-c // page_size) for c in ctxs) + 2
    kp = np.full((num_pages, nkv, page_size, d), 7.0)
    vp = np.full((num_pages, nkv, page_size, d), -9.0)
    free = list(rng.permutation(num_pages))
    tables = np.full((R, max_pages), -1, dtype=np.int32)
    rows, refs, new_kv = [], [], []
    def rotate(x, pos):   # [heads, d] at one position
        out = x.copy()
        c, s = np.cos(ang[pos])[None, :], np.sin(ang[pos])[None, :]
        out[:, :rot] = P.apply_rope(x[None, :, :rot], c, s)[0]
        return out
    for r, ctx in enumerate(ctxs):
        k = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))      # keys as stored: already rotated
        v = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))
        q_raw = as64(dev(rng.normal(size=(nq, d)), DT[dtype]))
        k_raw = as64(dev(rng.normal(size=(nkv, d)), DT[dtype]))
        pos = ctx - 1
        if write:
            k[pos] = as64(dev(rotate(k_raw, pos), DT[dtype]))         # what the kernel must store
            v_new = v[pos]
        for j in range(ctx):
            lp = j // page_size
            if tables[r, lp] < 0:
                tables[r, lp] = free.pop()
            if j == pos and write:
                continue                                                # left for the kernel to write
            kp[tables[r, lp], :, j % page_size] = k[j]
            vp[tables[r, lp], :, j % page_size] = v[j]
        q_rot = rotate(q_raw, pos)
        qfull = np.zeros((ctx, nq, d)); qfull[pos] = q_rot
        refs.append(P.attention(qfull, k, v, window=window)[pos].reshape(-1))
        rows.append(np.concatenate([q_raw.reshape(-1), k_raw.reshape(-1), v[pos].reshape(-1)]))
        new_kv.append((tables[r, pos // page_size], pos % page_size, k[pos], v[pos]))
    qkv = dev(np.array(rows), DT[dtype])
    dkp, dvp = dev(kp, DT[dtype]), dev(vp, DT[dtype])
    st = status()
    out = ops.decode_attention_fused(qkv, dkp, dvp, write, dev(tables, torch.int32),
                                     dev(np.arange(R + 1), torch.int32), dev(ctxs, torch.int32), cos_t, sin_t, rot,
                                     nq, nkv, d, 1 / math.sqrt(d), window, max_pos, st)
    assert int(st.item()) == 0
    ref = np.array(refs)
    assert rel_err(out, ref) < TOL[dtype] * (1 if dtype == "float32" else 1.5)
    for page, slot, k_want, v_want in new_kv:
        if write:
            assert np.abs(as64(dkp[page, :, slot]) - k_want).max() < TOL[dtype] * 4
            assert np.array_equal(as64(dvp[page, :, slot]), v_want)
    # twice in a row: the counters were left at zero
    out2 = ops.decode_attention_fused(qkv, dkp, dvp, write, dev(tables, torch.int32),
                                      dev(np.arange(R + 1), torch.int32), dev(ctxs, torch.int32), cos_t, sin_t, rot,
                                      nq, nkv, d, 1 / math.sqrt(d), window, max_pos, st)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("nq,nkv,d,rot,page_size,window,write", [
    (8, 2, 64, 64, 16, None, True), (32, 8, 64, 64, 16, None, True), (6, 2, 64, 64, 16, None, True),
    (24, 8, 128, 128, 16, None, True), (8, 2, 64, 32, 8, None, True), (8, 2, 64, 64, 16, 100, True),
    (4, 4, 128, 128, 4, 129, True), (16, 1, 64, 64, 32, None, True), (8, 2, 64, 64, 16, None, False),
    (12, 2, 64, 64, 16, 1100, True),
    # head size 128 fetches whole pages by TMA when a page has at least 8 rows: boxes of 8, 16 and 32 rows,
    # a window's edge inside a page, a layer that only reads the cache, a group of 16 heads
    (8, 2, 128, 128, 16, 100, True), (8, 2, 128, 64, 8, 1100, True), (16, 1, 128, 128, 64, None, True),
    (8, 2, 128, 128, 32, None, False)])
def test_tensor_core_decode_attention(nq, nkv, d, rot, page_size, window, write):
    """The cluster / tensor-core decode kernel against rotate-then-attend in float64;
    contexts from one token to several tiles per block (more than 8 tiles of 128)."""
    from kv_cache_optimization_for_llm_b200 import ops
    assert ops.decode_attention_mma_supported(d, nq // nkv, page_size)
    dtype = "bfloat16"
    rng = np.random.default_rng(nq * d + rot + page_size)
    ctxs = [1, 128, 129, 640, 300, 2, 1000, 2500, 1025]
    R = len(ctxs)
    max_pos = 2560
    inv = P.rope_inv_freq(rot, 10000.0)
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    cos_t, sin_t = dev(np.cos(ang), torch.float32), dev(np.sin(ang), torch.float32)
    max_pages = max(-(-c // page_size) for c in ctxs) + 1
    num_pages = sum(-(-c // page_size) for c in ctxs) + 2
    kp = np.full((num_pages, nkv, page_size, d), 7.0)
    vp = np.full((num_pages, nkv, page_size, d), -9.0)
    free = list(rng.permutation(num_pages))
    tables = np.full((R, max_pages), -1, dtype=np.int32)
    rows, refs, new_kv = [], [], []
    def rotate(x, pos):
        out = x.copy()
        c, s = np.cos(ang[pos])[None, :], np.sin(ang[pos])[None, :]
        out[:, :rot] = P.apply_rope(x[None, :, :rot], c, s)[0]
        return out
    for r, ctx in enumerate(ctxs):
        k = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))
        v = as64(dev(rng.normal(size=(ctx, nkv, d)), DT[dtype]))
        q_raw = as64(dev(rng.normal(size=(nq, d)), DT[dtype]))
        k_raw = as64(dev(rng.normal(size=(nkv, d)), DT[dtype]))
        pos = ctx - 1
        if write:
            k[pos] = as64(dev(rotate(k_raw, pos), DT[dtype]))
        for j in range(ctx):
            lp = j // page_size
            if tables[r, lp] < 0:
                tables[r, lp] = free.pop()
            if j == pos and write:
                continue
            kp[tables[r, lp], :, j % page_size] = k[j]
            vp[tables[r, lp], :, j % page_size] = v[j]
        q_rot = as64(dev(rotate(q_raw, pos), DT[dtype]))     # the kernel rounds the rotated query to bfloat16
        qfull = np.zeros((ctx, nq, d)); qfull[pos] = q_rot
        refs.append(P.attention(qfull, k, v, window=window)[pos].reshape(-1))
        rows.append(np.concatenate([q_raw.reshape(-1), k_raw.reshape(-1), v[pos].reshape(-1)]))
        new_kv.append((tables[r, pos // page_size], pos % page_size, k[pos], v[pos]))
    qkv = dev(np.array(rows), DT[dtype])
    dkp, dvp = dev(kp, DT[dtype]), dev(vp, DT[dtype])
    st = status()
    args = (qkv, dkp, dvp, write, dev(tables, torch.int32), dev(np.arange(R + 1), torch.int32),
            dev(ctxs, torch.int32), cos_t, sin_t, rot, nq, nkv, d, 1 / math.sqrt(d), window, st)
    out4 = ops.decode_attention_mma(*args, max_ctx=max(ctxs))      # the launch sized for the longest context here
    assert rel_err(out4, np.array(refs)) < TOL[dtype] * 1.5
    out = ops.decode_attention_mma(*args)                          # sized for any context
    # the classes a token's tiles fall into follow from its own position, not from the launch
    assert torch.equal(out, out4)
    assert int(st.item()) == 0
    assert rel_err(out, np.array(refs)) < TOL[dtype] * 1.5
    for page, slot, k_want, v_want in new_kv:
        if write:
            assert np.abs(as64(dkp[page, :, slot]) - k_want).max() < TOL[dtype] * 4
            assert np.array_equal(as64(dvp[page, :, slot]), v_want)
    assert torch.equal(out, ops.decode_attention_mma(*args))
    # a request's result does not depend on its neighbours in the batch: bit for bit
    one = ops.decode_attention_mma(qkv[3:4].contiguous(), dkp, dvp, write, dev(tables[3:4], torch.int32),
                                   dev([0, 1], torch.int32), dev(ctxs[3:4], torch.int32), cos_t, sin_t, rot, nq, nkv, d,
                                   1 / math.sqrt(d), window, st)
    assert torch.equal(one[0], out[3])
    # ... nor on the size of the batch, which decides how many blocks share a request's classes
    # of tiles: the same requests many times over (a large grid, clusters of 1 or 2 blocks)
    reps = 12
    big = (qkv.repeat(reps, 1), dkp, dvp, write, dev(np.tile(tables, (reps, 1)), torch.int32),
           dev(np.arange(R * reps + 1), torch.int32), dev(ctxs * reps, torch.int32), cos_t, sin_t, rot, nq, nkv, d,
           1 / math.sqrt(d), window, st)
    assert torch.equal(ops.decode_attention_mma(*big), out.repeat(reps, 1))
    assert torch.equal(ops.decode_attention_mma(*big, max_ctx=max(ctxs)), out4.repeat(reps, 1))
    assert int(st.item()) == 0


def test_tensor_core_decode_attention_long_contexts():
    """Contexts beyond 8192 tokens: 16 classes of tiles and clusters of 16 blocks.  No rotary
    encoding here, the cache already holds every key; one key far back is made to stand out."""
    from kv_cache_optimization_for_llm_b200 import ops
    nq, nkv, d, page_size = 8, 2, 64, 16
    rng = np.random.default_rng(5)
    ctxs = [8200, 12001, 70, 2049, 16500]
    R = len(ctxs)
    max_pages = max(-(-c // page_size) for c in ctxs) + 1
    num_pages = sum(-(-c // page_size) for c in ctxs) + 2
    kp = np.zeros((num_pages, nkv, page_size, d))
    vp = np.zeros((num_pages, nkv, page_size, d))
    free = list(rng.permutation(num_pages))
    tables = np.full((R, max_pages), -1, dtype=np.int32)
    rows, refs = [], []
    for r, ctx in enumerate(ctxs):
        k = as64(dev(rng.normal(size=(ctx, nkv, d)), torch.bfloat16))
        v = as64(dev(rng.normal(size=(ctx, nkv, d)), torch.bfloat16))
        q = as64(dev(rng.normal(size=(nq, d)), torch.bfloat16))
        far = ctx // 3                                     # this key gets a large score for head 0
        k[far, 0] = as64(dev(q[0] * 1.5, torch.bfloat16))
        for j in range(ctx):
            lp = j // page_size
            if tables[r, lp] < 0:
                tables[r, lp] = free.pop()
        idx = np.arange(ctx)
        kp[tables[r, idx // page_size], :, idx % page_size] = k
        vp[tables[r, idx // page_size], :, idx % page_size] = v
        out = np.zeros((nq, d))
        for h in range(nq):
            s_ = k[:, h // (nq // nkv)] @ q[h] / math.sqrt(d)
            p = np.exp(s_ - s_.max()); p /= p.sum()
            out[h] = p @ v[:, h // (nq // nkv)]
        refs.append(out.reshape(-1))
        # the row brings the newest key and value again; write_kv is off, so they are not used
        rows.append(np.concatenate([q.reshape(-1), k[ctx - 1].reshape(-1), v[ctx - 1].reshape(-1)]))
    qkv = dev(np.array(rows), torch.bfloat16)
    dkp, dvp = dev(kp, torch.bfloat16), dev(vp, torch.bfloat16)
    st = status()
    args = (qkv, dkp, dvp, False, dev(tables, torch.int32), dev(np.arange(R + 1), torch.int32), dev(ctxs, torch.int32),
            None, None, 0, nq, nkv, d, 1 / math.sqrt(d), None, st)
    out = ops.decode_attention_mma(*args, max_ctx=max(ctxs))
    assert int(st.item()) == 0
    assert rel_err(out, np.array(refs)) < TOL["bfloat16"] * 1.5
    # a launch sized for any context, and one request alone: the same bits
    assert torch.equal(out, ops.decode_attention_mma(*args))
    one = ops.decode_attention_mma(qkv[1:2].contiguous(), dkp, dvp, False, dev(tables[1:2], torch.int32),
                                   dev([0, 1], torch.int32), dev(ctxs[1:2], torch.int32), None, None, 0, nq, nkv, d,
                                   1 / math.sqrt(d), None, st, max_ctx=ctxs[1])
    assert torch.equal(one[0], out[1])


@pytest.mark.parametrize("d,nq,nkv,window,ctx", [(64, 8, 2, None, 9001), (64, 8, 2, 5000, 9100), (64, 32, 2, None, 8300),
                                                 (128, 8, 2, None, 8500), (128, 8, 2, 3000, 9000)])
def test_tensor_core_decode_attention_one_request_long_context(d, nq, nkv, window, ctx):
    """One request beyond 8192 tokens, alone in its launch (the form with two tiles in shared memory per block).
    The new key and value come with the row and are written to the cache by the kernel; under a window the new
    key's tile is among the first of its class, so it is also placed into its stage by hand.  One key far back
    (inside the window) stands out, one just outside it must not be seen.  The same request ten times in one
    launch takes the form with one tile per block: same bits."""
    from kv_cache_optimization_for_llm_b200 import ops
    page_size = 16
    rng = np.random.default_rng(ctx + d)
    G = nq // nkv
    k = as64(dev(rng.normal(size=(ctx, nkv, d)), torch.bfloat16))
    v = as64(dev(rng.normal(size=(ctx, nkv, d)), torch.bfloat16))
    q = as64(dev(rng.normal(size=(nq, d)), torch.bfloat16))
    lo = 0 if window is None else max(0, ctx - window)
    far = lo + 1
    k[far, 0] = as64(dev(q[0] * 1.5, torch.bfloat16))
    if window is not None:
        k[lo - 1, 0] = as64(dev(q[0] * 3.0, torch.bfloat16))    # just outside the window: must not be seen
    n_pages = -(-ctx // page_size)
    table = rng.permutation(n_pages + 3)[:n_pages].astype(np.int32)
    kp = np.zeros((n_pages + 3, nkv, page_size, d))
    vp = np.zeros((n_pages + 3, nkv, page_size, d))
    idx = np.arange(ctx - 1)                                    # the cache holds all but the newest
    kp[table[idx // page_size], :, idx % page_size] = k[:-1]
    vp[table[idx // page_size], :, idx % page_size] = v[:-1]
    ref = np.zeros((nq, d))
    for h in range(nq):
        s_ = k[lo:, h // G] @ q[h] / math.sqrt(d)
        pr = np.exp(s_ - s_.max()); pr /= pr.sum()
        ref[h] = pr @ v[lo:, h // G]
    row = np.concatenate([q.reshape(-1), k[-1].reshape(-1), v[-1].reshape(-1)])
    st = status()

    def run(reps):
        dkp, dvp = dev(kp, torch.bfloat16), dev(vp, torch.bfloat16)
        out = ops.decode_attention_mma(
            dev(np.tile(row, (reps, 1)), torch.bfloat16), dkp, dvp, True, dev(np.tile(table, (reps, 1)), torch.int32),
            dev(np.arange(reps + 1), torch.int32), dev([ctx] * reps, torch.int32), None, None, 0, nq, nkv, d,
            1 / math.sqrt(d), window, st, max_ctx=ctx)
        return out, dkp, dvp

    out, dkp, dvp = run(1)
    assert int(st.item()) == 0
    assert rel_err(out[0], ref.reshape(-1)) < TOL["bfloat16"]
    pos = ctx - 1
    assert torch.equal(dkp[int(table[pos // page_size]), :, pos % page_size].double().cpu(), torch.from_numpy(k[-1]))
    assert torch.equal(dvp[int(table[pos // page_size]), :, pos % page_size].double().cpu(), torch.from_numpy(v[-1]))
    many, _, _ = run(10)
    assert torch.equal(many, out.repeat(10, 1))


@pytest.mark.parametrize("d,nq,nkv", [(64, 8, 2), (128, 6, 2)])
@pytest.mark.parametrize("window", [100, 129])
@pytest.mark.parametrize("inside", [False, True])
def test_window_edge_with_a_key_that_stands_out(d, nq, nkv, window, inside):
    """The window's edge in the bfloat16 tensor-core kernels, shown by one key whose score
    stands out for the newest query: at position ``pos - window`` it must be ignored, at
    ``pos - window + 1`` it must be found.  One key too many or too few changes the newest
    row's output from "the mean of a hundred values" to "that key's value" or back.  A
    37-token portion whose rows straddle a key tile and a page edge (every prompt kernel),
    and the single newest token (the decode kernel)."""
    from kv_cache_optimization_for_llm_b200 import ops
    ctx, page_size = 900, 16
    pos = ctx - 1
    spike = pos - window + (1 if inside else 0)
    scale = 1 / math.sqrt(d)
    c = _attention_case("bfloat16", nq, nkv, d, ctxs=[ctx], q_lens=[37], page_size=page_size, window=window,
                        seed=d + window + inside, spike=spike)
    page, slot = int(c["table"][0, spike // page_size]), spike % page_size
    spike_value = np.repeat(as64(c["vp"][page, :, slot]), nq // nkv, axis=0).reshape(-1)
    # the plain result itself shows the difference: the newest row is that key's value, or far from it
    assert (np.abs(c["ref"][-1] - spike_value).max() < 0.05) == inside
    forms = [False, True, 3] + ([2] if d == 64 else [])
    for wide in forms:
        fb = _FakeBatch(c)
        out = ops.flash_attention(c["qkv"], c["kp"], c["vp"], c["table"], fb, nq, nkv, d, scale, window, wide=wide)
        assert int(fb.status.item()) == 0
        assert rel_err(out, c["ref"]) < TOL["bfloat16"], wide
        assert (np.abs(as64(out)[-1] - spike_value).max() < 0.08) == inside, wide
    one = _attention_case("bfloat16", nq, nkv, d, ctxs=[ctx], q_lens=[1], page_size=page_size, window=window,
                          seed=d + window + inside, spike=spike)
    st = status()
    out = ops.decode_attention_mma(one["qkv"], one["kp"], one["vp"], False, one["table"], one["q_start"],
                                   one["ctx_len"], None, None, 0, nq, nkv, d, scale, window, st, max_ctx=ctx)
    assert int(st.item()) == 0
    assert rel_err(out, one["ref"]) < TOL["bfloat16"] * 1.5
    assert (np.abs(as64(out)[-1] - spike_value).max() < 0.08) == inside


def test_decode_attention_wait_gives_up_and_the_context_stays_usable():
    """The waits of the page-by-page (TMA) decode attention are bounded: on barriers that nothing completes one
    warp runs out of polls, the kernel reports it and returns, the block's other warp leaves through the flag;
    afterwards the same context computes as before."""
    from kv_cache_optimization_for_llm_b200 import ops
    st = status()
    flags = ops.decode_wait_selftest(3000, st)
    torch.cuda.synchronize()
    assert int(st.item()) == 4 and "wait" in ops.STATUS_TEXT[4].lower()
    assert flags.tolist() == [1, 0]
    st.zero_()
    x = torch.arange(64, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum().item()) == 2 * 63 * 64 / 2 and int(st.item()) == 0


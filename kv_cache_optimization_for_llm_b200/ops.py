"""Python face of the CUDA kernels: loads each kernel module through ctypes at its
first use (building it if needed) and wraps the launchers.

There is no fallback: on a machine with a GPU a missing or unbuildable library
raises, and no operator here has a PyTorch or CPU stand-in.  Matrix products of
the bfloat16 path are this package's tcgen05 kernels for steps of up to 32 rows and,
from 128 rows, for the gate|up product (``KVB200_WIDE=all``: for every product); the
others go to the library (cuBLAS through ``torch.nn.functional.linear``) as all of
upstream's do (cublasGemmEx, base/src/engine.cu:653-671).  Everything else, and
every matrix product of the float32 path, is a kernel of this package.
"""

from __future__ import annotations

import collections
import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from typing import Dict, Optional

import torch

from . import build

_libs: Dict[str, ctypes.CDLL] = {}
launch_count = 0  # kernels of this package launched so far (library calls are not counted)
# Which kernel the dispatch below picked, how often (a launch that is captured into a graph counts
# once, at capture): what a test reads to see that the path it means to check is the one that ran.
choices: "collections.Counter[str]" = collections.Counter()

_ERR = {-1: "unsupported dtype", -2: "a size this kernel refuses", -3: "misaligned pointer or stride"}

STATUS_TEXT = {
    1: "a kernel met a position whose cache page is not mapped",
    2: "a kernel met a position outside the position-encoding table",
    3: "a kernel met a token id outside the vocabulary",
    4: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    pass


def lib(name: str) -> ctypes.CDLL:
    got = _libs.get(name)
    if got is None:
        build.ensure_built([name])
        path = build.kernel_lib_path(name)
        try:
            got = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"the kernel library {path} cannot be loaded: {e}") from e
        _libs[name] = got
    return got


def prepare(names) -> None:
    """Builds (in parallel) and loads the named kernel modules."""
    build.ensure_built(list(names))
    for n in names:
        lib(n)


def loaded_libraries():
    return {n: str(build.kernel_lib_path(n)) for n in _libs}


def _check(rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        if rc < 0:
            raise KernelError(f"{what}: {_ERR.get(rc, rc)}")
        raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")
    launch_count += 1


_step_stream: Optional[c_void_p] = None     # the stream of the running forward pass, looked up once
_step_capturing: Optional[bool] = None


class use_current_stream:
    """While active, the operators launch on the stream that was current at entry (and know whether
    it is being captured) without asking torch at every launch: the lookup costs 15 us, a step
    of a small model has a hundred launches."""

    def __enter__(self):
        global _step_stream, _step_capturing
        self.before = (_step_stream, _step_capturing)
        _step_stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        _step_capturing = torch.cuda.is_current_stream_capturing()
        return self

    def __exit__(self, *exc):
        global _step_stream, _step_capturing
        _step_stream, _step_capturing = self.before
        return False


def _stream() -> c_void_p:
    return _step_stream if _step_stream is not None else c_void_p(torch.cuda.current_stream().cuda_stream)


def _capturing() -> bool:
    return _step_capturing if _step_capturing is not None else torch.cuda.is_current_stream_capturing()


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_sm_count: Dict[int, int] = {}


def sm_count(device) -> int:
    """SMs of the device (asked once): what the dispatch compares a step's tiles with."""
    idx = torch.device(device).index or 0
    if idx not in _sm_count:
        _sm_count[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_count[idx]


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return 0
    if dt == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {dt} has no kernels (float32 and bfloat16 do)")


_arena = None      # the running step's arena (engine/arena.py), None outside a step


class use_arena:
    """While active, the tensors that the operators below produce come out of ``arena``
    instead of the allocator."""

    def __init__(self, arena):
        self.arena = arena

    def __enter__(self):
        global _arena
        self.before, _arena = _arena, self.arena
        return self.arena

    def __exit__(self, *exc):
        global _arena
        _arena = self.before
        return False


def new(shape, dtype: torch.dtype, device) -> torch.Tensor:
    """An uninitialised result tensor: out of the running step's arena when there is one (on
    its device), otherwise from the allocator (operators called on their own)."""
    a = _arena
    if a is not None and a.device == device:
        return a.new(shape, dtype)
    return torch.empty(tuple(shape), dtype=dtype, device=device)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of this package run on CUDA tensors only; there is no CPU path")


# ------------------------------------------------------------------ elementwise

def embed_gather(table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
                 sampled: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 residual rows ``table[ids]``.  With ``sampled`` (int32), an id ``-(1 + r)``
    stands for ``sampled[r]``: a token that is still on the device."""
    _need_cuda(table, ids, sampled)
    assert sampled is None or (sampled.dtype == torch.int32 and sampled.is_contiguous())
    V, H = table.shape
    T = ids.numel()
    out = new((T, H), torch.float32, table.device)
    rc = lib("elementwise").kvb_embed_gather(_p(table), dtype_code(table.dtype), _p(ids), _p(sampled),
                                             c_int(0 if sampled is None else sampled.numel()), _p(out),
                                             c_int(T), c_int(H), c_int(V), _p(status), _stream())
    _check(rc, "embed_gather")
    return out


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``resid += delta`` (when given, in float32, in place unless ``rows`` selects),
    then RMSNorm of the sum times ``weight`` (no weight: ``None``); ``rows`` (int32) picks the rows to
    produce, in order, leaving ``resid`` untouched."""
    _need_cuda(resid)
    assert resid.dtype == torch.float32 and resid.is_contiguous()
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == resid.shape[1])
    T, H = resid.shape
    n = T if rows is None else rows.numel()
    out = new((n, H), out_dtype, resid.device)
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    rc = lib("elementwise").kvb_add_rmsnorm(_p(resid), _p(delta), _p(weight), _p(out), _p(rows), c_int(n),
                                            c_int(H), c_float(eps), c_int(dtype_code(out_dtype)), _stream())
    _check(rc, "add_rmsnorm")
    return out


def silu_mul(gate_up: torch.Tensor, block: Optional[int] = None) -> torch.Tensor:
    """``silu(gate) * up`` for rows that hold gate and up in alternating blocks of
    ``block`` features ([gate | up] as a whole when ``block`` is None)."""
    _need_cuda(gate_up)
    assert gate_up.is_contiguous()
    T, two_i = gate_up.shape
    I = two_i // 2
    out = new((T, I), gate_up.dtype, gate_up.device)
    rc = lib("elementwise").kvb_silu_mul(_p(gate_up), _p(out), c_int(T), c_int(I), c_int(block or I),
                                         c_int(dtype_code(gate_up.dtype)), _stream())
    _check(rc, "silu_mul")
    return out


def rope_kv_write(qkv, positions, token_req, cos, sin, k_pages, v_pages, block_table, page_size,
                  nq, nkv, d, rot, status) -> None:
    """Rotates q (in place) and k, writes k and v into their pages.  ``k_pages`` None:
    only q is rotated.  ``cos`` None: no rotation."""
    _need_cuda(qkv)
    assert qkv.is_contiguous() and qkv.shape[1] == (nq + 2 * nkv) * d
    T = qkv.shape[0]
    table_len = 0 if cos is None else cos.shape[0]
    num_pages = 0 if k_pages is None else k_pages.shape[0]
    if k_pages is not None:
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == qkv.dtype
        assert tuple(k_pages.shape[1:]) == (nkv, page_size, d), (k_pages.shape, nkv, page_size, d)
    max_pages = block_table.shape[1]
    rc = lib("elementwise").kvb_rope_kv_write(
        _p(qkv), _p(positions), _p(token_req), _p(cos), _p(sin), c_int(table_len), _p(k_pages),
        _p(v_pages), _p(block_table), c_int(max_pages), c_int(page_size), c_int(num_pages), c_int(T),
        c_int(nq), c_int(nkv), c_int(d), c_int(rot), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "rope_kv_write")


# ------------------------------------------------------------------ attention

def paged_attention_generic(qkv, k_pages, v_pages, block_table, positions, token_req, nq, nkv, d,
                            scale, window, status) -> torch.Tensor:
    """Attention of every token in ``qkv`` (q part) over its request's cached keys."""
    _need_cuda(qkv, k_pages)
    T = qkv.shape[0]
    out = new((T, nq * d), qkv.dtype, qkv.device)
    page_size = k_pages.shape[2]
    rc = lib("attention").kvb_paged_attention_generic(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table),
        c_int(block_table.shape[1]), c_int(page_size), c_int(k_pages.shape[0]), _p(positions),
        _p(token_req), _p(out), c_int(T), c_int(nq), c_int(nkv), c_int(d), c_float(scale),
        c_int(int(window or 0)), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "paged_attention_generic")
    choices["paged_attention_generic"] += 1
    return out


# ------------------------------------------------------------------ matrix products

SKINNY_MAX_ROWS = int(os.environ.get('KVB200_SKINNY_MAX_ROWS', '32'))   # measured: the library product wins beyond
_status_word: Dict[int, torch.Tensor] = {}


def kernel_status(device) -> torch.Tensor:
    """The device word into which kernels report impossible indices and waits that ran
    out; one per device, shared by every engine in the process."""
    idx = torch.device(device).index or 0
    t = _status_word.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_word[idx] = t
    return t


class Folded:
    """What a product hands on in place of its output once it has added that output into
    the float32 residual itself: ``xb``, the new residual rows in bfloat16, and ``sumsq``
    [rows, parts], partial sums of their squares, from which the next norm's 1/rms follows."""
    __slots__ = ("xb", "sumsq")

    def __init__(self, xb: torch.Tensor, sumsq: torch.Tensor):
        self.xb, self.sumsq = xb, sumsq


class PendingNorm:
    """A weightless RMSNorm that has not been carried out (the norm's weight has been
    multiplied into the matrices that read its result): the float32 rows, their bfloat16
    copy and partial sums of squares, and eps.  ``linear`` and ``linear_swiglu`` take it in
    place of a tensor: they multiply the bare rows and scale each row of the result by its
    1/rms.  ``materialize`` runs the norm as a kernel of its own for everything else."""
    __slots__ = ("resid", "xb", "sumsq", "eps", "dtype")

    def __init__(self, resid, xb, sumsq, eps, dtype):
        self.resid, self.xb, self.sumsq, self.eps, self.dtype = resid, xb, sumsq, eps, dtype

    @property
    def shape(self):
        return self.resid.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.resid, None, None, self.eps, self.dtype)


FUSED_NORM = os.environ.get('KVB200_FUSED_NORM', '1') != '0'


def fused_norm_rows(rows: int, dtype: torch.dtype) -> bool:
    """Whether products over ``rows`` rows fold the residual add and the norm into themselves."""
    return FUSED_NORM and dtype == torch.bfloat16 and rows <= min(SKINNY_MAX_ROWS, FUSED_EPILOGUE_MAX_ROWS)


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, into: Optional[torch.Tensor] = None):
    """``x . w^T`` with ``w`` [out, in].
    float32: this package's FMA kernel (true 32-bit).
    bfloat16, few rows (decode and short portions): this package's tcgen05/TMA
    kernel, which streams the weights.  bfloat16 with more rows (long prompt portions):
    the library product, float32 accumulation, as upstream's cublasGemmEx.

    ``x`` may be a :class:`PendingNorm`.  ``into``: a float32 residual [rows, out] the
    caller is going to add the result to; where the tensor-core kernel can, it adds the
    product there itself and a :class:`Folded` comes back instead of a tensor."""
    if isinstance(x, PendingNorm):
        if into is None and fused_norm_rows(x.xb.shape[0], x.dtype) and w.dtype == torch.bfloat16:
            return gemm_skinny_fused(x.xb, w, kernel_status(w.device), row_scale=x,
                                     x_is_static=_capturing())
        if (into is None and wide_fused_rows(x.xb.shape[0], x.dtype) and _wide_ok(x.xb, w, 8)
                and (out_dtype is None or out_dtype == x.dtype)):
            return gemm_wide(x.xb, w, kernel_status(w.device), row_scale=x)
        x = x.materialize()
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype
    if (into is not None and fused_norm_rows(M, x.dtype) and _skinny_ok(x, FUSED_EPILOGUE_MAX_ROWS) and N % 8 == 0
            and into.dtype == torch.float32 and into.shape == (M, N) and into.is_contiguous()):
        return gemm_skinny_fused(x, w, kernel_status(w.device), into=into,
                                 x_is_static=_capturing())
    if (into is not None and wide_fused_rows(M, x.dtype) and _wide_ok(x, w, 8) and into.dtype == torch.float32
            and into.shape == (M, N) and into.is_contiguous() and N % 4 == 0):
        return gemm_wide(x, w, kernel_status(w.device), into=into)
    if x.dtype == torch.float32:
        assert x.stride(1) == 1 and w.stride(1) == 1
        out = new((M, N), torch.float32, x.device)
        rc = lib("gemm_f32").kvb_sgemm_nt(_p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out),
                                          c_int(N), c_int(M), c_int(N), c_int(K), _stream())
        _check(rc, "sgemm_nt")
        choices["sgemm_nt"] += 1
        return out
    if M <= SKINNY_MAX_ROWS and K % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        return gemm_skinny(x, w, out_dtype or x.dtype, kernel_status(x.device),
                           x_is_static=_capturing())
    if WIDE == "all" and _wide_ok(x, w, 8) and (out_dtype is None or out_dtype == x.dtype):
        return gemm_wide(x, w, kernel_status(x.device))
    choices["library_product"] += 1
    return _library_product(x, w, out_dtype or x.dtype)


_mm_takes_out_with_dtype = True    # whether torch.mm accepts out= together with out_dtype= (found out at first use)


def _library_product(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``x . w^T`` by the library (cuBLAS, float32 accumulation), written into a tensor of the
    step's arena."""
    global _mm_takes_out_with_dtype
    out = new((x.shape[0], w.shape[0]), out_dtype, x.device)
    if out_dtype == x.dtype:
        return torch.matmul(x, w.t(), out=out)
    if _mm_takes_out_with_dtype:
        try:
            return torch.mm(x, w.t(), out_dtype=out_dtype, out=out)
        except (TypeError, RuntimeError, NotImplementedError):
            _mm_takes_out_with_dtype = False
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# Which products of steps with many rows run on this package's tcgen05 kernel (gemm_bf16_wide.cu):
#   "auto"  those it is faster for on a B200 at every number of rows: the gate|up product, whose
#           SiLU * up it does as its epilogue (at 2048 rows it is level with the library for the
#           others, at 512 rows the library's split of K wins for the down product)
#   "all"   every one (no library product in a bfloat16 step)
#   "off"   none (the library product, then the activation kernel)
WIDE = os.environ.get('KVB200_WIDE', 'auto')
WIDE_MIN_ROWS = 128
# From this many rows on the products of a step also take the residual add and the RMSNorm into
# themselves (as the products of few rows do), which makes every product of the step this
# package's: below it the library's split of K is the faster way through the narrow products.  0: never.
WIDE_FUSED_MIN_ROWS = int(os.environ.get('KVB200_WIDE_FUSED_MIN_ROWS', '0'))


def wide_fused_rows(rows: int, dtype: torch.dtype) -> bool:
    """Whether products over ``rows`` rows (many) fold the residual add and the norm into themselves."""
    return (FUSED_NORM and WIDE != "off" and WIDE_FUSED_MIN_ROWS > 0 and dtype == torch.bfloat16
            and rows >= WIDE_FUSED_MIN_ROWS)


def _wide_ok(x: torch.Tensor, w: torch.Tensor, n_multiple: int) -> bool:
    """Whether the tcgen05 kernel for steps of many rows takes this product."""
    return (x.shape[0] >= WIDE_MIN_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and w.shape[0] % n_multiple == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _skinny_ok(x: torch.Tensor, rows_limit: int) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] <= rows_limit and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, block: int) -> torch.Tensor:
    """``silu(x . gate^T) * (x . up^T)`` with gate and up stored as one matrix whose rows
    alternate in blocks of ``block`` features.  Few bfloat16 rows (SKINNY_MAX_ROWS) with blocks of 64:
    one kernel (the activation is the product's epilogue); otherwise product, then
    activation kernel."""
    I = gate_up.shape[0] // 2
    if isinstance(x, PendingNorm):
        if fused_norm_rows(x.xb.shape[0], x.dtype) and gate_up.dtype == torch.bfloat16:
            st, static = kernel_status(gate_up.device), _capturing()
            if block == 64 and gate_up.shape[0] % 128 == 0:
                return gemm_skinny_fused(x.xb, gate_up, st, row_scale=x, epilogue="swiglu", x_is_static=static)
            return silu_mul(gemm_skinny_fused(x.xb, gate_up, st, row_scale=x, x_is_static=static),
                            block=block if block != I else None)
        if wide_fused_rows(x.xb.shape[0], x.dtype) and block == 64 and _wide_ok(x.xb, gate_up, 128):
            return gemm_wide(x.xb, gate_up, kernel_status(gate_up.device), epilogue="swiglu", row_scale=x)
        x = x.materialize()
    if block == 64 and _skinny_ok(x, min(SKINNY_MAX_ROWS, FUSED_EPILOGUE_MAX_ROWS)) \
            and gate_up.shape[0] % 128 == 0:
        return gemm_skinny(x, gate_up, x.dtype, kernel_status(x.device),
                           x_is_static=_capturing(), epilogue="swiglu")
    if WIDE != "off" and block == 64 and _wide_ok(x, gate_up, 128):
        return gemm_wide(x, gate_up, kernel_status(x.device), epilogue="swiglu")
    return silu_mul(linear(x, gate_up), block=block if block != I else None)


_scratch: Dict[tuple, torch.Tensor] = {}


def scratch(key: tuple, shape, dtype, device) -> torch.Tensor:
    """A buffer that lives as long as the process, one per key: kernels that need
    global memory beyond their inputs and outputs get it here, so that captured
    graphs see fixed addresses and steps allocate nothing."""
    t = _scratch.get(key)
    if t is None or t.shape != tuple(shape):
        t = torch.empty(shape, dtype=dtype, device=device)
        _scratch[key] = t
    return t


def decode_key_blocks(max_positions: int):
    """(keys per block, number of blocks) of the split decode kernel for an engine that
    allows ``max_positions`` tokens: at most 64 blocks, 128 keys or a multiple."""
    kb = 128 * max(1, -(-max_positions // (128 * 64)))
    return kb, -(-max_positions // kb)


def decode_attention_supported(d: int, group: int) -> bool:
    return bool(lib("attention").kvb_decode_attention_supported(c_int(d), c_int(group)))


def decode_attention(qkv, k_pages, v_pages, block_table, q_start, ctx_len, nq, nkv, d, scale, window,
                     max_positions, status, reqs_capacity=None) -> torch.Tensor:
    """One query token per request, split over key blocks, all heads of a group together."""
    _need_cuda(qkv, k_pages)
    R = ctx_len.numel()
    T = qkv.shape[0]
    kb, nb = decode_key_blocks(max_positions)
    cap = max(R, reqs_capacity or 0)
    part_o = scratch(("dec_o", qkv.device.index, cap, nq, nb, d), (cap, nq, nb, d), torch.float32, qkv.device)
    part_ml = scratch(("dec_ml", qkv.device.index, cap, nq, nb), (cap, nq, nb, 2), torch.float32, qkv.device)
    out = new((T, nq * d), qkv.dtype, qkv.device)
    rc = lib("attention").kvb_decode_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len), _p(out), _p(part_o),
        _p(part_ml), c_int(R), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)),
        c_int(kb), c_int(nb), c_int(dtype_code(qkv.dtype)), _p(status), _stream())
    _check(rc, "decode_attention")
    global launch_count
    launch_count += 1  # split and combine
    return out


FLASH_WIDE = os.environ.get('KVB200_FLASH_WIDE', '1') != '0'
FLASH_TC = os.environ.get('KVB200_FLASH_TC', '1') != '0'
FLASH_TC_ROLES = os.environ.get('KVB200_FLASH_TC_ROLES', '1') != '0'


def flash_attention_supported(d: int, group: int, page_size: int) -> bool:
    if d not in (64, 128):      # answered here, so that a model of another head size never builds the module
        return False
    return bool(lib("flash_attention").kvb_flash_attention_supported(c_int(d), c_int(group), c_int(page_size)))


_tokens_per_tile: Dict[tuple, int] = {}


def flash_tokens_per_tile(group: int, wide: bool) -> int:
    """Query tokens in one tile of the tensor-core attention for prompt portions: 64 rows
    (``wide`` False) or 128 rows of (token, head of the group) pairs."""
    key = (int(group), bool(wide))
    if key not in _tokens_per_tile:
        _tokens_per_tile[key] = int(lib("flash_attention").kvb_flash_attention_tokens_per_tile(
            c_int(key[0]), c_int(1 if wide else 0)))
    return _tokens_per_tile[key]


def flash_tiles(batch, group: int, wide: bool) -> torch.Tensor:
    """The query tiles of a step for a group size: [n, 4] int32 rows (request row, first
    token row, tokens, 0), each tile holding consecutive tokens of one request.  Built
    once per step, group size and tile height, kept on the batch."""
    nt = flash_tokens_per_tile(group, bool(wide))
    ready = (getattr(batch, "tiles", None) or {}).get(nt)
    if ready is not None:
        return ready            # laid out with the batch's other arrays and copied with them
    cache = batch.host.setdefault("flash_tiles", {})
    got = cache.get(nt)
    if got is None:
        import numpy as np
        qs = batch.host["q_start"]
        rows = []
        for r in range(batch.num_reqs):
            a, b = int(qs[r]), int(qs[r + 1])
            starts = np.arange(a, b, nt, dtype=np.int32)
            tile = np.zeros((len(starts), 4), dtype=np.int32)
            tile[:, 0] = r
            tile[:, 1] = starts
            tile[:, 2] = np.minimum(nt, b - starts)
            rows.append(tile)
        host = torch.from_numpy(np.concatenate(rows)).pin_memory()
        got = host.to(batch.token_ids.device, non_blocking=True)
        cache[nt] = got
        cache[("host", nt)] = host   # keep the pinned source alive until the step is over
    return got


def flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window,
                    wide: Optional[bool] = None, skip_single: bool = False,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-core attention for steps with runs of query tokens (bfloat16).  ``wide``:
    False: 64 query rows per block (mma.sync); True: 128 rows (mma.sync); 2: 128 rows on
    tcgen05 with the scores in tensor memory (head size 64); 3: the same with roles (a TMA
    loader warp, two issuing warps, four softmax warps; head size 64 or 128, pages of at least
    8 rows); None:
    chosen from the step's size, the head size and the page size.  ``skip_single``: the step's
    leading single tokens (``batch.num_single``) are somebody else's: their tiles are left out.
    ``out``: where the rows go; made here if not given."""
    _need_cuda(qkv, k_pages)
    skip = int(batch.num_single) if skip_single else 0
    T = qkv.shape[0] - skip
    # 128-row tiles when there are enough of them to keep every SM busy, else 64-row tiles
    nt128 = flash_tokens_per_tile(nq // nkv, True)
    if wide is None:
        # 128-row tiles when they fill the GPU: two blocks per SM at head size 64, one at 128
        wide = FLASH_WIDE and (T // nt128) * nkv >= (2 if d == 64 else 1) * sm_count(qkv.device)
        if wide and FLASH_TC:
            roles = (FLASH_TC_ROLES and k_pages.shape[2] >= 8 and k_pages.data_ptr() % 16 == 0
                     and v_pages.data_ptr() % 16 == 0 and qkv.data_ptr() % 16 == 0 and qkv.stride(0) % 8 == 0)
            if roles:
                wide = 3
            elif d == 64:
                wide = 2
    tiles = flash_tiles(batch, nq // nkv, wide)[skip:]      # a single token is one tile, and they come first
    if out is None:
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
    rc = lib("flash_attention").kvb_paged_flash_attention(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), _p(block_table), c_int(block_table.shape[1]),
        c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(batch.positions), _p(tiles), c_int(tiles.shape[0]),
        c_int(int(wide)), _p(out), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)), _p(batch.status),
        _stream())
    _check(rc, "paged_flash_attention")
    choices[f"flash_attention_{int(wide)}"] += 1
    return out


def decode_attention_fused(qkv, k_pages, v_pages, write_kv, block_table, q_start, ctx_len, cos, sin, rot,
                           nq, nkv, d, scale, window, max_positions, status, trace=None) -> torch.Tensor:
    """The whole attention of a decode step in one launch: rotary encoding of query and
    new key, the write of key and value into their page, split attention, merge."""
    _need_cuda(qkv, k_pages)
    R = ctx_len.numel()
    T = qkv.shape[0]
    kb, nb = decode_key_blocks(max_positions)
    dev = qkv.device
    part_o = scratch(("dec_o", dev.index, R, nq, nb, d), (R, nq, nb, d), torch.float32, dev)
    part_ml = scratch(("dec_ml", dev.index, R, nq, nb), (R, nq, nb, 2), torch.float32, dev)
    counters = _scratch.get(("dec_counters", dev.index))
    if counters is None or counters.numel() < R * nkv:
        counters = torch.zeros(max(R * nkv, 4096), dtype=torch.int32, device=dev)
        _scratch[("dec_counters", dev.index)] = counters
    out = new((T, nq * d), qkv.dtype, dev)
    rc = lib("attention").kvb_decode_attention_fused(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), c_int(1 if write_kv else 0), _p(block_table),
        c_int(block_table.shape[1]), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len),
        _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rot), _p(out), _p(part_o), _p(part_ml),
        _p(counters), c_int(R), c_int(nq), c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)),
        c_int(kb), c_int(nb), c_int(dtype_code(qkv.dtype)), _p(status), _p(trace), _stream())
    _check(rc, "decode_attention_fused")
    choices["decode_attention_fused"] += 1
    return out


def decode_attention_mma_supported(d: int, group: int, page_size: int) -> bool:
    if d not in (64, 128):      # answered here, so that a model of another head size never builds the module
        return False
    return bool(lib("decode_attention").kvb_decode_attention_mma_supported(c_int(d), c_int(group), c_int(page_size)))


def decode_context_class(max_ctx: int) -> int:
    """The classes of 128-key tiles (4, 8 or 16) that the longest context of a decode step
    needs in the tensor-core decode attention.  The launch (kernel variant, blocks per request)
    depends on it, the results do not; steps are replayed from graphs captured per class."""
    from .engine.batch import CONTEXT_CLASS_BOUNDS as bounds   # the block tables' widths follow the same classes
    return 4 if max_ctx <= bounds[0] else (8 if max_ctx <= bounds[1] else 16)


def decode_launch_context(batch) -> int:
    """The context length a decode step's launches are sized for: the upper end of the class
    of the step's longest context, so that every step of a class launches alike (a captured
    graph is replayed for all of them)."""
    from .engine.batch import CONTEXT_CLASS_BOUNDS as bounds
    c = decode_context_class(int(batch.max_ctx_len))
    return bounds[0] if c == 4 else (bounds[1] if c == 8 else 1 << 30)


def decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table, q_start, ctx_len, cos, sin, rot,
                         nq, nkv, d, scale, window, status, max_ctx: int = 0,
                         trace: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The attention of a bfloat16 decode step in one launch on tensor cores: rotary
    encoding of query and new key, cache write, attention over 128-key tiles spread over
    a cluster of blocks, merge through distributed shared memory.  No scratch.
    A token's tiles fall into 4 classes below position 2048, 8 below 8192, 16 beyond (head
    size 64), whatever the batch; up to that many blocks share a (request, kv head).
    ``max_ctx``: the longest context of the step if the host knows it (the launch is sized
    for it), 0 otherwise.  ``out``: where the rows go ([tokens, nq d], the rows of the requests'
    tokens are written); made here if not given."""
    _need_cuda(qkv, k_pages)
    assert qkv.dtype == torch.bfloat16
    R = ctx_len.numel()
    if out is None:
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
    rc = lib("decode_attention").kvb_decode_attention_mma(
        _p(qkv), c_int(qkv.stride(0)), _p(k_pages), _p(v_pages), c_int(1 if write_kv else 0), _p(block_table),
        c_int(block_table.shape[1]), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), _p(q_start), _p(ctx_len),
        _p(cos), _p(sin), c_int(0 if cos is None else cos.shape[0]), c_int(rot), _p(out), c_int(R), c_int(nq),
        c_int(nkv), c_int(d), c_float(scale), c_int(int(window or 0)), c_int(int(max_ctx)),
        _p(status), _p(trace), _stream())
    _check(rc, "decode_attention_mma")
    choices["decode_attention_mma"] += 1
    return out


def attention_step(qkv, k_pages, v_pages, write_kv, block_table, batch, nq, nkv, d, scale, window, max_positions,
                   cos, sin, rot) -> torch.Tensor:
    """Everything between the q|k|v projection and the output projection: rotary
    encoding, the write of keys and values into their pages, attention over the pages.
    Picks the kernels:
    * float32: rotary/write kernel, then the general kernel, whose sums follow absolute
      positions in one fixed order whatever the shape of the step;
    * bfloat16, single tokens only: one fused launch, on tensor cores where the sizes allow
      (head size 64/128), else the FMA form (head size 32);
    * bfloat16, runs of tokens: rotary/write kernel, then the tensor-core kernel; single tokens
      beside them (they are the step's first rows) go to the fused launch of decode steps;
    * sizes neither takes: rotary/write kernel, then the general kernel."""
    group, page_size = nq // nkv, k_pages.shape[2]
    if qkv.dtype == torch.bfloat16 and batch.decode_only and decode_attention_mma_supported(d, group, page_size):
        return decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table, batch.q_start, batch.ctx_len,
                                    cos, sin, rot, nq, nkv, d, scale, window, batch.status,
                                    max_ctx=decode_launch_context(batch))
    if qkv.dtype == torch.bfloat16 and batch.decode_only and decode_attention_supported(d, group):
        return decode_attention_fused(qkv, k_pages, v_pages, write_kv, block_table, batch.q_start, batch.ctx_len,
                                      cos, sin, rot, nq, nkv, d, scale, window, max_positions, batch.status)
    ns = int(getattr(batch, "num_single", 0))
    if (qkv.dtype == torch.bfloat16 and ns > 0 and flash_attention_supported(d, group, page_size)
            and decode_attention_mma_supported(d, group, page_size)):
        # Single tokens beside runs: the single tokens (the step's first rows) go to the kernel of
        # decode steps, which rotates, writes and attends in one launch, the runs to the two kernels
        # for runs.  As a tile of the kernel for runs a single token would fill 4 of 128 rows.
        out = new((qkv.shape[0], nq * d), qkv.dtype, qkv.device)
        decode_attention_mma(qkv, k_pages, v_pages, write_kv, block_table[:ns], batch.q_start[:ns + 1], batch.ctx_len[:ns],
                             cos, sin, rot, nq, nkv, d, scale, window, batch.status,
                             max_ctx=decode_launch_context(batch), out=out)
        rope_kv_write(qkv[ns:], batch.positions[ns:], batch.token_req[ns:], cos, sin, k_pages if write_kv else None,
                      v_pages if write_kv else None, block_table, page_size, nq, nkv, d, rot, batch.status)
        return flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window,
                               skip_single=True, out=out)
    rope_kv_write(qkv, batch.positions, batch.token_req, cos, sin, k_pages if write_kv else None,
                  v_pages if write_kv else None, block_table, page_size, nq, nkv, d, rot, batch.status)
    if qkv.dtype == torch.bfloat16 and not batch.decode_only and flash_attention_supported(d, group, page_size):
        return flash_attention(qkv, k_pages, v_pages, block_table, batch, nq, nkv, d, scale, window)
    return paged_attention_generic(qkv, k_pages, v_pages, block_table, batch.positions, batch.token_req,
                                   nq, nkv, d, scale, window, batch.status)


# ------------------------------------------------------------------ sampling

def sample(logits, temperature, seed, key, pos, penalty, mask, slots, out=None, status=None,
           status_at: int = 0) -> torch.Tensor:
    """One token id per row of float32 ``logits``.  ``temperature`` None: greedy for all
    rows; ``penalty``/``mask`` None: no repetition penalty.  ``status``: the kernels' error
    word, copied to ``out[status_at]`` so that it travels with the tokens."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    R, V = logits.shape
    if out is None:
        out = new((R,), torch.int32, logits.device)
    rc = lib("sampling").kvb_sample(_p(logits), c_int(R), c_int(V), _p(temperature), _p(seed), _p(key),
                                    _p(pos), _p(penalty), _p(mask), _p(slots), _p(out), _p(status),
                                    c_int(status_at), _stream())
    _check(rc, "sample")
    return out


def reset_mask(mask: torch.Tensor, slot: int, tokens: Optional[torch.Tensor]) -> None:
    """Clears the slot's row of produced-token marks and marks ``tokens`` (int32, device)."""
    n = 0 if tokens is None else tokens.numel()
    rc = lib("sampling").kvb_reset_mask(_p(mask), c_int(slot), c_int(mask.shape[1]), _p(tokens), c_int(n),
                                        _stream())
    _check(rc, "reset_mask")


# ------------------------------------------------------------------ bfloat16 matrix products (tcgen05)

def gemm_skinny_plan(M: int, N: int, K: int):
    """(blocks along K, tiles along N) of the skinny tensor-core kernel, or None if it
    does not take the sizes."""
    splits, tiles = c_int(0), c_int(0)
    rc = lib("gemm_bf16").kvb_gemm_skinny_plan(c_int(M), c_int(N), c_int(K), ctypes.byref(splits), ctypes.byref(tiles))
    if rc != 0:
        return None
    return splits.value, tiles.value


FUSED_EPILOGUE_MAX_ROWS = int(os.environ.get('KVB200_FUSED_MAX_ROWS', '32'))   # the kernel takes up to 64


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, status: torch.Tensor,
                x_is_static: bool = False, trace: Optional[torch.Tensor] = None, epilogue: str = "store") -> torch.Tensor:
    """``x . w^T`` for few rows (M <= 256) on tcgen05 tensor cores, weights streamed by TMA.

    ``epilogue``: "store", or "swiglu": ``w`` holds gate and up rows in alternating blocks
    of 64 and ``silu(gate) * up`` [M, N/2] is returned (up to 64 rows)."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    code = {"store": 0, "swiglu": 1}[epilogue]
    out = new((M, N // 2 if code == 1 else N), out_dtype, x.device)
    rc = lib("gemm_bf16").kvb_gemm_skinny(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(1 if out_dtype == torch.float32 else 0),
        c_int(M), c_int(N), c_int(K), c_int(1 if x_is_static else 0), c_int(code), _p(status), _p(trace),
        _stream())
    if rc == -2:
        raise KernelError(f"gemm_skinny refuses M={M}, N={N}, K={K} (M <= 256 and K a multiple of 8 are required)")
    _check(rc, "gemm_skinny")
    choices["gemm_skinny"] += 1
    return out


def gemm_skinny_fused(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor, row_scale: Optional[PendingNorm] = None,
                      into: Optional[torch.Tensor] = None, epilogue: str = "store", x_is_static: bool = False,
                      trace: Optional[torch.Tensor] = None):
    """The skinny product (up to 64 rows) with the residual stream's add and RMSNorm folded around it.

    ``row_scale``: every row of ``x . w^T`` is multiplied by the 1/rms that follows from the
    pending norm's partial sums (``x`` is then its bare bfloat16 rows, and ``w`` has the
    norm's weight multiplied into its columns).  ``into``: the product is added into this
    float32 residual in place and a :class:`Folded` is returned; otherwise the product
    (``epilogue`` "store" or "swiglu") as a bfloat16 tensor."""
    _need_cuda(x, w)
    N, K = w.shape
    M = x.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    assert x.shape[1] == K and M <= 64
    ss, parts, eps = None, 0, 0.0
    if row_scale is not None:
        ss, eps = row_scale.sumsq, row_scale.eps
        assert into is None and ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape[0] == M
        parts = ss.shape[1]
    out = sumsq = xb = None
    if into is not None:
        assert epilogue == "store" and into.dtype == torch.float32 and into.shape == (M, N) and into.stride(1) == 1
        code = 2
        sumsq = new((M, -(-N // 128)), torch.float32, x.device)
        xb = new((M, N), torch.bfloat16, x.device)
    else:
        code = {"store": 0, "swiglu": 1}[epilogue]
        out = new((M, N // 2 if code == 1 else N), torch.bfloat16, x.device)
    rc = lib("gemm_bf16").kvb_gemm_skinny_fused(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(M), c_int(N), c_int(K),
        c_int(1 if x_is_static else 0), c_int(code), _p(ss), c_int(parts), c_float(eps),
        _p(into), c_int(into.stride(0) if into is not None else 0), _p(xb), _p(sumsq), _p(status), _p(trace),
        _stream())
    if rc == -2:
        raise KernelError(f"gemm_skinny_fused refuses M={M}, N={N}, K={K}, epilogue {epilogue}")
    _check(rc, "gemm_skinny_fused")
    choices["gemm_skinny_fused"] += 1
    return Folded(xb, sumsq) if into is not None else out


def gemm_wide(x: torch.Tensor, w: torch.Tensor, status: torch.Tensor, epilogue: str = "store",
              tile=(0, 0), row_scale: Optional[PendingNorm] = None, into: Optional[torch.Tensor] = None):
    """``x . w^T`` for steps of many rows on tcgen05 tensor cores: a persistent kernel with a TMA
    loader warp, an issuing warp and four epilogue warps, two accumulators in tensor memory.

    ``epilogue``: "store", or "swiglu": ``w`` holds gate and up rows in alternating blocks
    of 64 and ``silu(gate) * up`` [M, N/2] is returned.  ``tile``: (rows of x, features) per
    tile, one of (128, 64), (128, 128), (128, 256), (256, 256); (256, 256, 1): such a tile shared
    by the two blocks of a cluster; (0, 0) for the kernel's own choice.

    ``row_scale``: every row of ``x . w^T`` is multiplied by the 1/rms that follows from the
    pending norm's partial sums (``x`` is then its bare bfloat16 rows, and ``w`` has the
    norm's weight multiplied into its columns).  ``into``: the product is added into this
    float32 residual in place and a :class:`Folded` is returned."""
    _need_cuda(x, w)
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    assert w.shape[1] == K
    ss, parts, eps = None, 0, 0.0
    if row_scale is not None:
        ss, eps = row_scale.sumsq, row_scale.eps
        assert into is None and ss.dtype == torch.float32 and ss.is_contiguous() and ss.shape[0] == M
        parts = ss.shape[1]
    out = xb = sumsq = None
    if into is not None:
        assert epilogue == "store" and into.dtype == torch.float32 and into.shape == (M, N) and into.stride(1) == 1
        code = 2
        sumsq = new((M, -(-N // 256)), torch.float32, x.device)
        xb = new((M, N), torch.bfloat16, x.device)
    else:
        code = {"store": 0, "swiglu": 1}[epilogue]
        out = new((M, N // 2 if code == 1 else N), torch.bfloat16, x.device)
    rc = lib("gemm_bf16_wide").kvb_gemm_wide_fused(
        _p(x), c_int(x.stride(0)), _p(w), c_int(w.stride(0)), _p(out), c_int(out.stride(0) if out is not None else 0),
        c_int(M), c_int(N), c_int(K), c_int(code), c_int(tile[0]), c_int(tile[1]),
        c_int(tile[2] if len(tile) > 2 else 0), _p(ss), c_int(parts), c_float(eps), _p(into),
        c_int(into.stride(0) if into is not None else 0), _p(xb), _p(sumsq), _p(status), _stream())
    if rc in (-2, -3):
        raise KernelError(f"gemm_wide refuses M={M}, N={N}, K={K}, epilogue {epilogue}, tile {tile} (K and N "
                          "multiples of 8, N a multiple of 128 for swiglu, 16-byte aligned rows are required)")
    _check(rc, "gemm_wide")
    choices["gemm_wide"] += 1
    return Folded(xb, sumsq) if into is not None else out


def wait_selftest(polls: int, status: torch.Tensor) -> None:
    """Lets the product kernels' bounded barrier wait run out on a barrier that nothing
    completes: ``status`` receives the wait-timeout code, the kernel returns."""
    rc = lib("gemm_bf16").kvb_wait_selftest(ctypes.c_uint(int(polls)), _p(status), _stream())
    _check(rc, "wait_selftest")


def decode_wait_selftest(polls: int, status: torch.Tensor) -> torch.Tensor:
    """Runs the decode attention's bounded wait (head size 128 waits for its pages on mbarriers) against barriers
    that nothing completes: one warp gives up after ``polls`` polls, reports KVB_STATUS_WAIT_TIMEOUT in ``status``
    and raises the block's flag, by which the other warp leaves.  Returns [flag, whether the other warp's wait
    claimed success] as an int32 tensor."""
    flags = torch.full((2,), -1, dtype=torch.int32, device=status.device)
    rc = lib("decode_attention").kvb_decode_wait_selftest(ctypes.c_uint(int(polls)), _p(status), _p(flags), _stream())
    _check(rc, "decode_wait_selftest")
    return flags

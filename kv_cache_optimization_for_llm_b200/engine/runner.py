"""Loads a model folder and runs steps on it: the one step function of the engine.

``step`` takes a batch of (request, its next tokens): portions of prompts beside
single decoded tokens, cut anywhere.  It runs only the tokens it is given, as one
batch, against the cache that earlier steps left, and returns the logits at the
wanted places.  Upstream has two separate passes instead, whole packed prompts
(prefillBatch, base/src/engine.cu:550-979) and one token per running sequence
(decodeStep, base/src/engine.cu:982-1311), and returns sampled ids only.
"""

from __future__ import annotations

import gc
from pathlib import Path
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..cache.paged_cache import PagedCache
from ..config import EngineConfig, read_config_json
from ..models.spec import expected_weights
from ..parts import BuildContext
from ..registry import resolve_architecture
from ..weights.loader import check_and_load
from .batch import BatchBuilder, StepBatch, StepEntry
from .model import DecoderModel

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class CacheFull(RuntimeError):
    """The pool has too few free pages for the step."""


def _require_gpu(device: torch.device) -> None:
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA device only (its kernels are built for sm_100a); "
                           "no GPU is visible and there is no CPU path")


class ModelRunner:
    def __init__(self, model_dir, config: Optional[EngineConfig] = None, random_init: Optional[dict] = None):
        """``model_dir``: folder with config.json and model.safetensors.  Or
        ``random_init={"config": <config.json dict>, "seed": s, "std": sd}`` with
        ``model_dir=None``: the same model with random weights drawn on the device,
        nothing written to disk."""
        self.config = config or EngineConfig()
        self.device = torch.device(self.config.device)
        _require_gpu(self.device)
        torch.cuda.set_device(self.device)
        # float32 means float32: no reduced-precision matrix mode anywhere.
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        # bfloat16 library products add up in float32 whatever the split of K (upstream:
        # CUBLAS_COMPUTE_32F, base/src/engine.cu:653-671)
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.model_dir = Path(model_dir) if model_dir is not None else None
        if self.model_dir is None and not random_init:
            raise ValueError("a model folder or random_init is required")
        config_dict = read_config_json(self.model_dir) if self.model_dir is not None else dict(random_init["config"])
        self.arch = resolve_architecture(config_dict)
        self.model_config = self.arch.parse_config(config_dict)
        self.spec = self.arch.build_spec(self.model_config)
        self.dtype = _TORCH_DTYPE[self.config.dtype]
        # Compile, side by side, what this model needs and nothing else.
        from .. import build
        from .model import kernel_modules_of
        build.ensure_built(kernel_modules_of(self.spec, self.dtype) + ["_host"])
        if self.model_dir is not None:
            tensors = check_and_load(self.model_dir, expected_weights(self.spec))
        else:
            from ..weights.random_init import random_tensors_on_device
            tensors = random_tensors_on_device(expected_weights(self.spec), int(random_init.get("seed", 0)),
                                               float(random_init.get("std", 0.02)), self.dtype, self.device)
        self.weight_bytes = sum(int(t.numel()) * t.element_size() for t in tensors.values())
        self.graph_mixed_steps = (self.weight_bytes <= 4 << 30) if self.config.graph_mixed_steps is None \
            else bool(self.config.graph_mixed_steps)
        self.max_model_len = int(self.config.max_model_len or self.spec.max_position)
        if self.max_model_len > self.spec.max_position:
            raise ValueError(f"max_model_len {self.max_model_len} exceeds the model's "
                             f"max_position_embeddings {self.spec.max_position}")
        self.status = ops.kernel_status(self.device)
        ctx = BuildContext(dtype=self.dtype, device=self.device, max_positions=self.max_model_len,
                           status=self.status)
        self.model = DecoderModel(self.spec, tensors, ctx)
        del tensors
        ops.prepare(self.model.kernel_modules())
        specs, cache_of = self.model.cache_specs()
        num_pages = self.config.num_pages
        if num_pages is None:
            per_token = PagedCache.bytes_per_token(specs, cache_of, self.dtype)
            free, _total = torch.cuda.mem_get_info(self.device)
            if per_token == 0:
                num_pages = self.config.max_num_seqs
            else:
                num_pages = int(free * self.config.memory_fraction) // (per_token * self.config.page_size)
                # More pages than every seat at full length can use are of no use.
                ceiling = self.config.max_num_seqs * (-(-self.max_model_len // self.config.page_size))
                num_pages = max(1, min(num_pages, ceiling))
        self.cache = PagedCache(specs, cache_of, self.config.page_size, num_pages, self.config.max_num_seqs,
                                self.max_model_len, self.dtype, self.device)
        self.manager = self.cache.manager
        self.builder = BatchBuilder(self.config.max_num_batched_tokens, self.config.max_num_seqs,
                                    self.cache.max_pages, self.device, self.status,
                                    page_size=self.config.page_size, tile_heights=self.model.query_tile_heights())
        # Everything a step computes lives here; steps allocate nothing.
        from .arena import StepArena
        self.arena = StepArena(self.device, *self.model.arena_bytes(self.config.max_num_batched_tokens,
                                                                     self.config.max_num_seqs))
        self.vocab_size = self.spec.vocab_size
        # Where the sampling kernel leaves a step's tokens (one per sampled request, in the
        # step's order; the last entry carries the kernels' error word).  A step whose entries
        # name tokens as -(1 + row) reads them from here.
        self.sampled = torch.zeros(self.config.max_num_seqs + 1, dtype=torch.int32, device=self.device)
        # Captured decode steps, by padded batch size.
        self._graphs = {}
        self._graph_pool = None
        self.graph_launches = 0   # kernels of this package launched through graph replays
        self.step_kinds = {"decode_graph": 0, "portion_graph": 0, "mixed_graph": 0, "launched": 0}   # how steps ran
        self.graph_buckets = []
        if self.config.use_cuda_graphs:
            b = 1
            while b < self.config.max_num_seqs:
                self.graph_buckets.append(b)
                b *= 2
            self.graph_buckets.append(self.config.max_num_seqs)
            if self.config.capture_graphs_at_start:
                self.capture_decode_graphs()

    # ---------------------------------------------------------------- the step function
    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs one batch whose pages are already in place.  Returns float32 logits
        [wanted, vocab] on the device, in the order of the entries and their ``want``."""
        if self.graph_buckets and all(len(e.tokens) == 1 for e in entries):
            self.step_kinds["decode_graph"] += 1
            return self._run_decode_graph(entries)
        if self.graph_buckets:
            runs = [e for e in entries if len(e.tokens) != 1]
            if len(runs) == 1:
                bucket = self._portion_bucket(runs[0])
                singles = len(entries) - 1
                if bucket and singles == 0:
                    self.step_kinds["portion_graph"] += 1
                    return self._run_portion_graph(entries[0], bucket)
                if bucket and self.graph_mixed_steps and len(entries) <= self.config.max_num_seqs:
                    rb = min(next(b for b in self.graph_buckets if b >= singles), self.config.max_num_seqs - 1)
                    if rb + bucket <= self.config.max_num_batched_tokens:
                        self.step_kinds["mixed_graph"] += 1
                        return self._run_mixed_graph(entries, runs[0], bucket, rb)
        self.step_kinds["launched"] += 1
        batch = self.builder.build(entries, self.manager, self.vocab_size, sampled=self.sampled[:-1])
        return self.model.forward(batch, self.cache, self.arena)

    # A step that is one request's portion of at most this many tokens is padded to the next of
    # these lengths and replayed from a captured graph: launched kernel by kernel it is bound by
    # the host (a hundred and fifty launches), which a prompt that arrives at an idle engine pays
    # as time to its first token.
    PORTION_BUCKETS = (16, 32, 64, 128, 256, 512)

    def _portion_bucket(self, e: StepEntry) -> int:
        n = len(e.tokens)
        if n < 2 or n > self.PORTION_BUCKETS[-1] or len(e.want) > 1 or self.cache.states or self.page_size_unknown():
            return 0
        bucket = next(b for b in self.PORTION_BUCKETS if b >= n)
        if bucket > self.config.max_num_batched_tokens or e.start + bucket > self.max_model_len:
            return 0
        if min(e.tokens) < 0:            # ids that name tokens still on the device belong to single tokens
            return 0
        return bucket

    def page_size_unknown(self) -> bool:
        return self.builder.page_size is None

    def _run_portion_graph(self, e: StepEntry, bucket: int) -> torch.Tensor:
        """One request's portion, padded with dummy tokens to ``bucket`` and replayed as a CUDA graph
        (captured at first use, one per bucket and width of the block tables)."""
        want = tuple(e.want) or (0,)
        batch = self.builder.build([StepEntry(e.request_id, e.tokens, e.start, want)], self.manager, self.vocab_size,
                                   scratch_page=self.cache.scratch_page, sampled=self.sampled[:-1], pad_tokens_to=bucket)
        key = ("portion", bucket, tuple(int(t.shape[1]) for t in batch.block_tables))
        got = self._graphs.get(key)
        if got is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.model.forward(batch, self.cache, self.arena)      # warm-up outside the capture
            torch.cuda.current_stream().wait_stream(side)
            before = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            gc.collect()                                               # see _run_decode_graph
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self.model.forward(batch, self.cache, self.arena)
            finally:
                if collecting:
                    gc.enable()
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            got = (graph, out, ops.launch_count - before, None)
            self._graphs[key] = got
            ops.launch_count = before
        graph, out, launches, _ = got
        graph.replay()
        self.graph_launches += launches
        return out[:1] if e.want else out[:0]

    def _run_mixed_graph(self, entries: Sequence[StepEntry], run: StepEntry, bucket: int, rb: int) -> torch.Tensor:
        """Single tokens beside one portion (a short prompt that arrives while others decode, the tail
        of a long one): the single tokens padded with dummy requests to a batch-size bucket as in
        ``_run_decode_graph``, the portion with dummy tokens as in ``_run_portion_graph``, replayed as
        one graph per (bucket of requests, bucket of tokens, width of the block tables).  The graph
        produces the logits of every single token and of one place of the portion; what was asked
        for is picked afterwards, in the order of the entries."""
        singles = [e for e in entries if e is not run]
        n_single = len(singles)
        # rb: the bucket of the single tokens' requests (at most max_num_seqs - 1: the portion's request is one too)
        asked = [StepEntry(e.request_id, e.tokens, e.start, (0,)) for e in singles]
        asked.append(StepEntry(run.request_id, run.tokens, run.start, tuple(run.want) or (0,)))
        batch = self.builder.build(asked, self.manager, self.vocab_size, pad_reqs_to=rb + 1,
                                   scratch_page=self.cache.scratch_page, scratch_slot=self.cache.scratch_slot,
                                   sampled=self.sampled[:-1], pad_tokens_to=bucket)
        key = ("mixed", rb, bucket, tuple(int(t.shape[1]) for t in batch.block_tables))
        got = self._graphs.get(key)
        if got is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.model.forward(batch, self.cache, self.arena)      # warm-up outside the capture
            torch.cuda.current_stream().wait_stream(side)
            before = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            gc.collect()                                               # see _run_decode_graph
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self.model.forward(batch, self.cache, self.arena)
            finally:
                if collecting:
                    gc.enable()
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            got = (graph, out, ops.launch_count - before, None)
            self._graphs[key] = got
            ops.launch_count = before
        graph, out, launches, _ = got
        graph.replay()
        self.graph_launches += launches
        # rows of `out`: the single tokens in their order, then the portion's place, then the dummies
        keep, k = [], 0
        for e in entries:
            if e is run:
                if e.want:
                    keep.append(n_single)
            else:
                if e.want:
                    keep.append(k)
                k += 1
        if keep == list(range(len(keep))):
            return out[:len(keep)]
        return out[keep] if keep else out[:0]

    def capture_decode_graphs(self) -> int:
        """Captures, before any request, the graph of every batch-size bucket for every class of
        context length that ``max_model_len`` allows, on dummy rows that read and write the
        scratch page only.  Returns how many graphs were captured.  Without it each graph is
        captured by the first step that needs it."""
        from .batch import CONTEXT_CLASS_BOUNDS
        before = len(self._graphs)
        contexts = [1] + [b + 1 for b in CONTEXT_CLASS_BOUNDS if b + 1 <= self.max_model_len]
        for ctx in contexts:
            for bucket in self.graph_buckets:
                self._run_decode_graph([], bucket=bucket, pad_ctx=ctx)
        torch.cuda.synchronize(self.device)
        self.status.zero_()
        return len(self._graphs) - before

    def _run_decode_graph(self, entries: Sequence[StepEntry], bucket: Optional[int] = None,
                          pad_ctx: int = 1) -> torch.Tensor:
        """A step of single tokens only: padded to the next captured batch size and
        replayed as one CUDA graph (captured at first use).  The graph reads the
        batch arrays at their fixed device addresses; only their contents change."""
        n = len(entries)
        if bucket is None:
            bucket = next(b for b in self.graph_buckets if b >= n)
        wants = [bool(e.want) for e in entries]
        padded = [StepEntry(e.request_id, e.tokens, e.start, (0,)) for e in entries]
        batch = self.builder.build(padded, self.manager, self.vocab_size, pad_reqs_to=bucket,
                                   scratch_page=self.cache.scratch_page, scratch_slot=self.cache.scratch_slot,
                                   sampled=self.sampled[:-1], pad_ctx=pad_ctx)
        # one graph per padded batch size and class of context length (launches are sized by both)
        key = (bucket, ops.decode_context_class(batch.max_ctx_len))
        got = self._graphs.get(key)
        if got is None:
            # Every row's logits are produced; rows are picked after the replay.
            rows = torch.arange(bucket, dtype=torch.int32, device=self.device)
            batch.logit_rows, batch.num_logits = rows, bucket
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.model.forward(batch, self.cache, self.arena)      # warm-up outside the capture
            torch.cuda.current_stream().wait_stream(side)
            before = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            # The collector must not run inside the capture: if it finds an engine that is gone, it
            # destroys that engine's graphs, which CUDA refuses while a stream is capturing, and the
            # refusal ends this capture too.  What is garbage now is collected first.
            gc.collect()
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    out = self.model.forward(batch, self.cache, self.arena)
            finally:
                if collecting:
                    gc.enable()
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            got = (graph, out, ops.launch_count - before, rows)
            self._graphs[key] = got
            ops.launch_count = before                       # captured, not launched
        graph, out, launches, _rows = got
        graph.replay()
        self.graph_launches += launches
        if all(wants):
            return out[:n]
        keep = [i for i, w in enumerate(wants) if w]
        return out[keep] if keep else out[:0]

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """``run`` with the cache kept for the caller: admits unknown requests, takes
        the pages the step needs (or raises :class:`CacheFull` and changes nothing),
        and records the new lengths afterwards."""
        m = self.manager
        admitted: List[int] = []
        try:
            for e in entries:
                if not m.has(e.request_id):
                    if m.admit(e.request_id) < 0:
                        raise CacheFull(f"no state slot is free for request {e.request_id}")
                    admitted.append(e.request_id)
                if m.computed(e.request_id) != e.start:
                    raise ValueError(f"request {e.request_id}: the step starts at position {e.start}, "
                                     f"its cache holds {m.computed(e.request_id)} tokens")
                if e.start + len(e.tokens) > self.max_model_len:
                    raise ValueError(f"request {e.request_id} would grow to {e.start + len(e.tokens)} tokens, "
                                     f"beyond max_model_len {self.max_model_len}")
            need = [0] * m.num_groups()
            for e in entries:
                for g, n in enumerate(m.pages_needed(e.request_id, e.start + len(e.tokens))):
                    need[g] += n
            for g, n in enumerate(need):
                if n > m.free_pages(g):
                    raise CacheFull(f"the step needs {n} pages of group {g}, {m.free_pages(g)} are free")
            for e in entries:
                if not m.extend(e.request_id, e.start + len(e.tokens)):
                    raise CacheFull("pages ran out while extending")  # cannot happen after the count above
        except Exception:
            for rid in admitted:
                m.release(rid)
            raise
        logits = self.run(entries)
        for e in entries:
            m.advance(e.request_id, e.start + len(e.tokens))
        return logits

    def release(self, request_id: int) -> None:
        if self.manager.has(request_id):
            self.manager.release(request_id)

    def check_status(self, code: Optional[int] = None) -> None:
        """Raises if a kernel reported an impossible index since the last check.  ``code``:
        the status word as it came back with a step's tokens; without it the word is read
        from the device (which synchronises)."""
        if code is None:
            code = int(self.status.item())
        if code:
            self.status.zero_()
            raise ops.KernelError(ops.STATUS_TEXT.get(code, f"kernel status {code}"))

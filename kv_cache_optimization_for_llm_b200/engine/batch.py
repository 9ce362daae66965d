"""The description of one step's batch, as the kernels read it.

A step carries, for each scheduled request, a run of new tokens that starts where
its cache ends: a portion of a prompt, or one decoded token.  Upstream builds two
different sets of descriptor arrays, one for packed whole prompts and one for
decode rows (base/src/engine.cu:584-633,993-1032); here one layout serves both,
staged in a single pinned buffer and copied with one transfer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """One request's share of a step."""
    request_id: int
    tokens: Sequence[int]        # the new tokens, in order; -(1 + r) names the token that the
                                 # sampling kernel of the step before left in row r on the device
    start: int                   # position of tokens[0] in its sequence
    want: Sequence[int] = ()     # indices into ``tokens`` whose logits are asked for


@dataclass
class StepBatch:
    num_tokens: int
    num_reqs: int
    token_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32, index of each token in its own sequence
    token_req: torch.Tensor      # [T] int32, row of each token's request in this batch
    q_start: torch.Tensor        # [R+1] int32, first token of each request's run
    req_start: torch.Tensor      # [R] int32, position of the run's first token
    ctx_len: torch.Tensor        # [R] int32, tokens in the cache after this step
    slots: torch.Tensor          # [R] int32, state slot of each request
    block_tables: List[torch.Tensor]  # per cache group [R, max_pages] int32
    logit_rows: torch.Tensor     # [n] int32, token rows whose logits are wanted
    num_logits: int
    max_q_len: int
    max_ctx_len: int
    decode_only: bool            # every run is a single token
    status: torch.Tensor         # [1] int32 device word that kernels report into
    host: dict = field(default_factory=dict)  # numpy mirrors of the arrays above
    sampled: Optional[torch.Tensor] = None    # [n] int32 on the device: what ids below zero refer to
    tiles: dict = field(default_factory=dict)  # tokens per tile -> [n, 4] int32 query tiles (request row, first
                                               # token row, tokens, 0) for the heights the mixers asked for
    num_single: int = 0          # in a step that mixes single tokens with runs: the single tokens' requests come
                                 # first (rows 0 .. num_single-1 of the requests, of the tokens and of every list of tiles)


# Decode launches and captured graphs come in classes by the step's longest context (up to
# 2048 tokens, up to 8192, beyond); the block tables of a step are as wide as its class needs.
CONTEXT_CLASS_BOUNDS = (2048, 8192)


def table_columns(max_ctx_len: int, page_size: Optional[int], max_pages: int) -> int:
    """Columns of a step's block tables: the pages that the upper end of the class of the
    step's longest context spans, at most ``max_pages`` (all of them without a page size).
    Every step of a class has the same width, so the graph captured for the class fits all."""
    if page_size is None:
        return max_pages
    for bound in CONTEXT_CLASS_BOUNDS:
        if max_ctx_len <= bound:
            return max(1, min(max_pages, -(-bound // page_size)))
    return max_pages


class BatchBuilder:
    """Turns entries plus the cache manager's tables into device arrays.

    All arrays of one step live in one device buffer of fixed layout (so that a
    captured graph can read them at fixed addresses) and are staged in one pinned
    host buffer."""

    def __init__(self, max_tokens: int, max_reqs: int, max_pages_per_group: Sequence[int], device,
                 status: torch.Tensor, page_size: Optional[int] = None, tile_heights: Sequence[int] = ()):
        """``page_size``: tokens per cache page.  When it is given, a step's block tables are
        only as wide as the step's longest context needs (see :func:`table_columns`) and lie
        packed behind one another; without it they always have ``max_pages_per_group`` columns."""
        self.max_tokens, self.max_reqs = int(max_tokens), int(max_reqs)
        self.max_pages = [int(m) for m in max_pages_per_group]
        self.page_size = None if page_size is None else int(page_size)
        # Tokens per query tile that mixers cut a step's runs of tokens into (attention kernels for
        # prompt portions): the tiles of every height are laid out behind the block tables.
        self.tile_heights = sorted({int(h) for h in tile_heights if int(h) > 0})
        self.device = torch.device(device)
        self.status = status
        T, R = self.max_tokens, self.max_reqs
        # The arrays of a step lie packed behind one another, each only as long as the step needs,
        # so that one short copy carries a short step.  Where each lies is a function of the step's
        # numbers of tokens and requests and of the widths of its block tables only: a captured
        # graph, keyed by all of these, finds them again.
        off = self._place(T, R)[1]
        for mp in self.max_pages:
            off += (R * mp + 3) // 4 * 4
        for h in self.tile_heights:
            off += 4 * (T // h + R + 1)
        self.total = off
        use_cuda = self.device.type == "cuda"
        # Two pinned staging buffers, used in turn: the copy of one step may still be under
        # way while the next step is written.  Each buffer's event tells when its copy is over.
        self._staging = []
        for _ in range(2):
            buf = torch.zeros(self.total, dtype=torch.int32, pin_memory=use_cuda)
            self._staging.append({"buf": buf, "np": buf.numpy(),
                                  "event": torch.cuda.Event() if use_cuda else None, "busy": False})
        self._turn = 0
        self.dev_buf = torch.zeros(self.total, dtype=torch.int32, device=self.device)
        self.last_h2d_bytes = 0

    @staticmethod
    def _place(T: int, R: int):
        """Offsets of the per-token and per-request arrays of a step with T tokens and R requests
        (every array 16-byte aligned; the wanted rows get room for all T), and where the block
        tables start."""
        at, off = {}, 0
        for name, n in (("token_ids", T), ("positions", T), ("token_req", T), ("logit_rows", T),
                        ("q_start", R + 1), ("req_start", R), ("ctx_len", R), ("slots", R)):
            at[name] = off
            off += (n + 3) // 4 * 4
        return at, off

    def build(self, entries: Sequence[StepEntry], cache, vocab_size: Optional[int] = None,
              pad_reqs_to: int = 0, scratch_page: int = -1, scratch_slot: int = 0,
              sampled: Optional[torch.Tensor] = None, pad_ctx: int = 1, pad_tokens_to: int = 0) -> StepBatch:
        """``cache`` is the CacheManager; every entry's pages must already cover
        ``start + len(tokens)``.

        ``pad_reqs_to`` > len(entries) appends single-token dummy requests (token 0 at
        position 0, writing to ``scratch_page`` and ``scratch_slot``, which no real
        request owns) so that a decode batch fills a captured graph's fixed shape;
        their rows follow the real ones and their logits are never read.  ``pad_ctx`` > 1
        gives the dummy requests a context of that many tokens, all of it the scratch page
        (what a graph captured ahead of any request is shaped with).

        ``pad_tokens_to`` > the tokens of a step's only run (its only entry of more than one token;
        the others may be single tokens) appends dummy tokens (id 0) at the
        positions behind that run, so that a portion fills a captured graph's fixed shape: they
        attend to what lies before them, nothing real attends to them, and their keys and values
        go behind the request's length, into the rest of its last page and, beyond that, into
        ``scratch_page``, where the next real tokens overwrite them or nobody reads them.

        ``sampled``: the device buffer that token ids below zero refer to (see StepEntry);
        without it such ids are refused."""
        padded_run, padded_entry = 0, -1
        if pad_tokens_to:
            runs = [i for i, e in enumerate(entries) if len(e.tokens) != 1]
            if len(runs) != 1:
                raise ValueError("only a step with exactly one run of tokens can be padded with tokens")
            padded_entry = runs[0]
            e0 = entries[padded_entry]
            padded_run = max(0, pad_tokens_to - len(e0.tokens))
            if padded_run:
                entries = list(entries)
                entries[padded_entry] = StepEntry(e0.request_id, list(e0.tokens) + [0] * padded_run, e0.start, e0.want)
        n_real = len(entries)
        if pad_reqs_to > n_real:
            # dummy requests want their logits when the step also holds a run: the rows of logits of
            # a captured graph are as many as its requests, whichever of them are real
            entries = list(entries) + [StepEntry(-1, (0,), max(0, pad_ctx - 1), (0,) if pad_tokens_to else ())
                                       for _ in range(pad_reqs_to - n_real)]
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        if R == 0 or T == 0:
            raise ValueError("a step needs at least one token")
        if R > self.max_reqs:
            raise ValueError(f"a step holds {R} requests, the engine was built for {self.max_reqs}")
        if T > self.max_tokens:
            raise ValueError(f"a step holds {T} tokens, the engine was built for {self.max_tokens}")
        stage = self._staging[self._turn]
        self._turn ^= 1
        if stage["busy"]:
            stage["event"].synchronize()
            stage["busy"] = False
        h = stage["np"]
        at, tables_at = self._place(T, R)
        tok = h[at["token_ids"]:at["token_ids"] + T]
        pos = h[at["positions"]:at["positions"] + T]
        treq = h[at["token_req"]:at["token_req"] + T]
        qs = h[at["q_start"]:at["q_start"] + R + 1]
        rstart = h[at["req_start"]:at["req_start"] + R]
        ctx = h[at["ctx_len"]:at["ctx_len"] + R]
        slots = h[at["slots"]:at["slots"] + R]
        # A step that mixes single tokens (decoding requests) with runs of tokens (prompt portions)
        # is laid out with the single tokens first, so that a mixer can hand the first rows to the
        # kernel it has for single tokens and the rest to the one for runs.  The wanted logits keep
        # the order of the entries as the caller gave them.
        singles = [i for i, e in enumerate(entries) if len(e.tokens) == 1]
        mixed = 0 < len(singles) < R
        order = singles + [i for i, e in enumerate(entries) if len(e.tokens) != 1] if mixed else list(range(R))
        first_row = [0] * R              # of entry i, as given: the row of its first token
        t = 0
        for r, i in enumerate(order):
            e = entries[i]
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id} brings no token to this step")
            tok[t:t + n] = e.tokens
            pos[t:t + n] = np.arange(e.start, e.start + n, dtype=np.int32)
            treq[t:t + n] = r
            qs[r] = t
            rstart[r] = e.start
            ctx[r] = e.start + n
            slots[r] = cache.slot_of(e.request_id) if i < n_real else scratch_slot
            first_row[i] = t
            t += n
        qs[R] = T
        rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"request {e.request_id}: wanted place {w} is outside its {len(e.tokens)} tokens")
                rows.append(first_row[i] + w)
        lowest = 0 if sampled is None else -int(sampled.numel())
        if vocab_size is not None and (tok.min() < lowest or tok.max() >= vocab_size):
            raise ValueError(f"a token id is outside the vocabulary of {vocab_size}")
        h[at["logit_rows"]:at["logit_rows"] + len(rows)] = rows
        max_ctx = int(ctx.max())
        widths = [table_columns(max_ctx, self.page_size, mp) for mp in self.max_pages]
        places, off = [], tables_at
        for g, cols in enumerate(widths):
            places.append(off)
            bt = h[off:off + R * cols].reshape(R, cols)
            bt.fill(-1)
            for r, i in enumerate(order):
                if i >= n_real:          # a dummy request: its context is the scratch page
                    bt[r, :max(1, min(cols, -(-pad_ctx // (self.page_size or pad_ctx))))] = scratch_page
                    continue
                e = entries[i]
                table = cache.block_table(e.request_id, g)
                if len(table) > self.max_pages[g]:
                    raise ValueError(f"request {e.request_id} holds {len(table)} pages in group {g}, "
                                     f"tables were sized for {self.max_pages[g]}")
                n = min(len(table), cols)      # pages beyond the step's longest context are not read
                bt[r, :n] = table[:n]
                if padded_run and i == padded_entry:   # the dummy tokens' pages behind the request's own
                    bt[r, n:min(cols, -(-(e.start + len(e.tokens)) // (self.page_size or 1)))] = scratch_page
            off += (R * cols + 3) // 4 * 4
        decode_only = all(len(e.tokens) == 1 for e in entries)
        tile_places = {}
        if not decode_only:
            for nt in self.tile_heights:
                n_tiles = 0
                for r, i in enumerate(order):
                    e = entries[i]
                    a, b = int(qs[r]), int(qs[r]) + len(e.tokens)
                    k = -(-(b - a) // nt)
                    tile = h[off + 4 * n_tiles:off + 4 * (n_tiles + k)].reshape(k, 4)
                    starts = np.arange(a, b, nt, dtype=np.int32)
                    tile[:, 0] = r
                    tile[:, 1] = starts
                    tile[:, 2] = np.minimum(nt, b - starts)
                    tile[:, 3] = 0
                    n_tiles += k
                tile_places[nt] = (off, n_tiles)
                off += 4 * n_tiles
        used = off      # tables and tiles lie last, so one copy of the used prefix carries everything
        self.dev_buf[:used].copy_(stage["buf"][:used], non_blocking=True)
        if stage["event"] is not None:
            stage["event"].record()
            stage["busy"] = True
        self.last_h2d_bytes = 4 * used
        d = self.dev_buf
        batch = StepBatch(
            num_tokens=T, num_reqs=R,
            token_ids=d[at["token_ids"]:at["token_ids"] + T], positions=d[at["positions"]:at["positions"] + T],
            token_req=d[at["token_req"]:at["token_req"] + T], q_start=d[at["q_start"]:at["q_start"] + R + 1],
            req_start=d[at["req_start"]:at["req_start"] + R], ctx_len=d[at["ctx_len"]:at["ctx_len"] + R],
            slots=d[at["slots"]:at["slots"] + R],
            block_tables=[d[o:o + R * cols].view(R, cols) for o, cols in zip(places, widths)],
            logit_rows=d[at["logit_rows"]:at["logit_rows"] + len(rows)], num_logits=len(rows),
            max_q_len=max(len(e.tokens) for e in entries),
            max_ctx_len=max_ctx,
            decode_only=decode_only,
            tiles={nt: d[o:o + 4 * n].view(n, 4) for nt, (o, n) in tile_places.items()},
            status=self.status,
            host={"q_start": qs.copy(), "ctx_len": ctx.copy(), "req_start": rstart.copy()},
            sampled=sampled,
            num_single=len(singles) if mixed else 0,
        )
        return batch

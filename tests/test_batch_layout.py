"""The arrays of a step as the kernels read them, built on the CPU: runs of tokens, positions,
wanted rows, block tables only as wide as the step's context class, query tiles of the heights
the mixers ask for, padding rows of a graph's fixed shape; and that short steps make short copies."""

import numpy as np
import torch

from kv_cache_optimization_for_llm_b200.engine.batch import BatchBuilder, StepEntry, table_columns


class _Manager:
    def __init__(self, tables, slots):
        self.tables, self.slots = tables, slots

    def slot_of(self, rid):
        return self.slots[rid]

    def block_table(self, rid, g):
        return self.tables[rid]


def _builder(**kw):
    return BatchBuilder(256, 8, [4096 // 16], torch.device("cpu"), torch.zeros(1, dtype=torch.int32), page_size=16, **kw)


def test_table_width_follows_the_context_class():
    assert table_columns(1, 16, 8192) == 128 and table_columns(2048, 16, 8192) == 128
    assert table_columns(2049, 16, 8192) == 512 and table_columns(8193, 16, 8192) == 8192
    assert table_columns(100, 16, 40) == 40 and table_columns(100, None, 40) == 40


def test_mixed_step_arrays_tables_and_tiles():
    b = _builder(tile_heights=[16, 32])
    m = _Manager({7: [5, 9, 2], 3: [11], 4: [8, 1, 6, 0, 13]}, {7: 2, 3: 0, 4: 1})
    batch = b.build([StepEntry(7, [10, 11, 12], 40, [2]), StepEntry(3, [99], 0, [0]),
                     StepEntry(4, list(range(50)), 20, [0, 49])], m, vocab_size=100)
    assert batch.num_tokens == 54 and batch.num_reqs == 3 and not batch.decode_only
    # the request that brings a single token comes first (a mixer hands it to its kernel for single
    # tokens), the runs follow in the order given
    assert batch.num_single == 1
    assert batch.token_ids.tolist() == [99, 10, 11, 12] + list(range(50))
    assert batch.positions.tolist() == [0, 40, 41, 42] + list(range(20, 70))
    assert batch.token_req.tolist() == [0] + [1] * 3 + [2] * 50
    assert batch.q_start.tolist() == [0, 1, 4, 54] and batch.ctx_len.tolist() == [1, 43, 70]
    assert batch.req_start.tolist() == [0, 40, 20] and batch.slots.tolist() == [0, 2, 1]
    # the wanted rows keep the caller's order: request 7's third token, request 3's token, request 4's first and last
    assert batch.logit_rows.tolist() == [3, 0, 4, 53] and batch.num_logits == 4
    assert batch.max_ctx_len == 70 and batch.max_q_len == 50
    bt = batch.block_tables[0]
    assert tuple(bt.shape) == (3, 128)          # the class of contexts up to 2048 tokens, not all 256 columns
    assert bt[1, :4].tolist() == [5, 9, 2, -1] and bt[0, :2].tolist() == [11, -1] and bt[2, :6].tolist() == [8, 1, 6, 0, 13, -1]
    # query tiles: consecutive tokens of one request, at most `height` each; the single tokens' tiles first
    assert batch.tiles[16].tolist() == [[0, 0, 1, 0], [1, 1, 3, 0], [2, 4, 16, 0], [2, 20, 16, 0], [2, 36, 16, 0], [2, 52, 2, 0]]
    assert batch.tiles[32].tolist() == [[0, 0, 1, 0], [1, 1, 3, 0], [2, 4, 32, 0], [2, 36, 18, 0]]
    # a step of runs only, or of single tokens only, keeps the order given
    runs = b.build([StepEntry(7, [10, 11, 12], 40, [2]), StepEntry(4, [1, 2], 20, [])], m, vocab_size=100)
    assert runs.num_single == 0 and runs.token_ids.tolist() == [10, 11, 12, 1, 2]
    batch = b.build([StepEntry(7, [10, 11, 12], 40, [2]), StepEntry(3, [99], 0, [0]),
                     StepEntry(4, list(range(50)), 20, [0, 49])], m, vocab_size=100)
    # everything lies packed in one buffer: the copy is a few hundred integers, not the engine's capacity
    assert b.last_h2d_bytes < 4 * (4 * 56 + 3 * 4 + 4 + 3 * 128 + 4 * 10 + 64)
    assert b.last_h2d_bytes < 4 * b.total // 3


def test_decode_step_padding_rows_and_fixed_places():
    b = _builder(tile_heights=[16])
    m = _Manager({1: [3, 4], 2: [7]}, {1: 0, 2: 1})
    entries = [StepEntry(1, [5], 17, [0]), StepEntry(2, [-1], 3, [0])]
    sampled = torch.zeros(8, dtype=torch.int32)
    one = b.build(entries, m, 100, pad_reqs_to=4, scratch_page=77, scratch_slot=8, sampled=sampled)
    assert one.decode_only and one.num_reqs == 4 and not one.tiles
    assert one.token_ids.tolist() == [5, -1, 0, 0] and one.ctx_len.tolist() == [18, 4, 1, 1]
    assert one.slots.tolist() == [0, 1, 8, 8]
    bt = one.block_tables[0]
    assert bt[2, :2].tolist() == [77, -1] and bt[3, 0].item() == 77 and bt[0, :3].tolist() == [3, 4, -1]
    assert b.last_h2d_bytes <= 4 * (4 * 4 + 8 + 3 * 4 + 4 * 128)
    # another step of the same shape finds every array at the same place (what a captured graph relies on)
    two = b.build([StepEntry(2, [9], 4, [0])], m, 100, pad_reqs_to=4, scratch_page=77, scratch_slot=8, sampled=sampled)
    for name in ("token_ids", "positions", "q_start", "ctx_len", "slots", "logit_rows"):
        assert getattr(one, name).data_ptr() == getattr(two, name).data_ptr(), name
    assert one.block_tables[0].data_ptr() == two.block_tables[0].data_ptr()
    # dummy requests with a context of their own (graphs captured ahead of any request)
    far = b.build([], m, 100, pad_reqs_to=2, scratch_page=77, scratch_slot=8, sampled=sampled, pad_ctx=2049)
    assert far.ctx_len.tolist() == [2049, 2049] and far.positions.tolist() == [2048, 2048]
    assert tuple(far.block_tables[0].shape) == (2, 256)       # the class up to 8192 tokens, capped by the 256 pages of this engine
    assert far.block_tables[0][0, :130].tolist() == [77] * 129 + [-1]


def test_random_steps_keep_every_request_together_and_the_wanted_rows_in_order():
    """Random steps (single tokens and runs in any order, with and without the padding of a graph's
    fixed shape): every request's tokens stay together and in order, the single tokens' requests come
    first when runs are present, the wanted rows follow the order of the entries as given, dummy
    requests and dummy tokens only ever name the scratch page, and real tables are copied unchanged."""
    rng = np.random.default_rng(123)
    page = 16
    for trial in range(200):
        n_req = int(rng.integers(1, 7))
        n_runs = int(rng.integers(0, 3)) if n_req > 1 else int(rng.integers(0, 2))
        kinds = ["run"] * min(n_runs, n_req) + ["single"] * (n_req - min(n_runs, n_req))
        rng.shuffle(kinds)
        pad_tokens = kinds.count("run") == 1 and rng.random() < 0.5
        pad_reqs = (pad_tokens or kinds.count("run") == 0) and rng.random() < 0.5
        entries, tables, slots = [], {}, {}
        for i, kind in enumerate(kinds):
            rid = 100 + i
            n = 1 if kind == "single" else int(rng.integers(2, 40))
            start = int(rng.integers(0, 300))
            toks = rng.integers(1, 90, n).tolist()
            want = sorted(set(rng.integers(0, n, int(rng.integers(0, 3))).tolist())) if not pad_tokens else [n - 1]
            entries.append(StepEntry(rid, toks, start, want))
            tables[rid] = (1000 + 50 * i + np.arange(-(-(start + n) // page))).tolist()
            slots[rid] = i
        b = _builder(tile_heights=[16])
        kw = {}
        run_len = next((len(e.tokens) for e in entries if len(e.tokens) != 1), 0)
        if pad_tokens:
            kw["pad_tokens_to"] = 64 if run_len <= 64 else 0
            pad_tokens = bool(kw["pad_tokens_to"])
        if pad_reqs:
            kw["pad_reqs_to"] = 8
        batch = b.build(entries, _Manager(tables, slots), vocab_size=100, scratch_page=7777, scratch_slot=99, **kw)
        R = batch.num_reqs
        qs, ctx, treq = batch.q_start.tolist(), batch.ctx_len.tolist(), batch.token_req.tolist()
        toks, pos = batch.token_ids.tolist(), batch.positions.tolist()
        assert treq == sorted(treq) and qs[-1] == batch.num_tokens            # requests' tokens together, rows ascending
        lens = [qs[r + 1] - qs[r] for r in range(R)]
        if any(n != 1 for n in lens) and any(n == 1 for n in lens):
            first_run = next(r for r in range(R) if lens[r] != 1)
            assert all(n != 1 for n in lens[first_run:]) and batch.num_single == first_run   # single tokens first
        else:
            assert batch.num_single == 0
        # every real entry is found again, whole and in order, with its table and slot
        row_of = {}
        for e in entries:
            r = next(r for r in range(R) if batch.slots[r].item() == slots[e.request_id] and batch.req_start[r].item() == e.start
                     and toks[qs[r]:qs[r] + len(e.tokens)] == list(e.tokens))
            row_of[e.request_id] = r
            assert pos[qs[r]:qs[r] + len(e.tokens)] == list(range(e.start, e.start + len(e.tokens)))
            n_pages = len(tables[e.request_id])
            assert batch.block_tables[0][r, :n_pages].tolist() == tables[e.request_id]
            rest = batch.block_tables[0][r, n_pages:].tolist()
            padded = lens[r] - len(e.tokens)
            assert padded == (kw.get("pad_tokens_to", 0) - len(e.tokens) if pad_tokens and len(e.tokens) != 1 else 0)
            extra = -(-(e.start + lens[r]) // page) - n_pages if padded else 0
            assert rest[:max(0, extra)] == [7777] * max(0, extra) and all(x == -1 for x in rest[max(0, extra):])
            assert ctx[r] == e.start + lens[r]
        # the wanted rows, in the order of the entries as given (dummy requests' rows follow when they want any)
        want_rows = [qs[row_of[e.request_id]] + w for e in entries for w in e.want]
        assert batch.logit_rows.tolist()[:len(want_rows)] == want_rows
        # dummy requests: one token each, the scratch page and slot
        for r in set(range(R)) - set(row_of.values()):
            assert lens[r] == 1 and batch.slots[r].item() == 99 and batch.block_tables[0][r, 0].item() == 7777

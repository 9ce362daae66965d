"""The scheduler's decisions, with the native cache manager and no model: admission in
order, prompts cut under the token budget, decode beside prefill, finishing, and what
happens when pages run out (the latest arrival is dropped, goes to the queue's front,
and is recomputed; a request too large for the pool ends with an error)."""

import random

import pytest

from kv_cache_optimization_for_llm_b200.cache import host_runtime

H = host_runtime()


def make(pages=16, page_size=4, slots=4, seqs=4, budget=16, model_len=64, chunk=0):
    cache = H.CacheManager([H.GroupSpec(page_size, 0)], [pages], slots)
    return cache, H.Scheduler(cache, H.SchedulerConfig(seqs, budget, model_len, chunk))


def run_step(sched, token_of=lambda rid, pos: (rid * 31 + pos) % 97, stop=None):
    plan = sched.schedule()
    sched.commit(plan)
    out = []
    for e in plan.entries:
        if e.sample:
            tok = token_of(e.id, e.start + len(e.tokens))
            reason = sched.append_token(e.id, tok, stop is not None and tok == stop)
            out.append((e.id, tok, reason))
    return plan, out


def test_prompt_is_cut_under_the_budget_and_decode_goes_first():
    cache, s = make(budget=8)
    s.add(0, list(range(20)), 4)
    plan, _ = run_step(s)
    assert [(e.id, e.start, len(e.tokens), e.sample) for e in plan.entries] == [(0, 0, 8, False)]
    s.add(1, list(range(5)), 4)
    plan, _ = run_step(s)     # request 0 continues (8 more), nothing left for request 1
    assert [(e.id, e.start, len(e.tokens)) for e in plan.entries] == [(0, 8, 8)]
    plan, out = run_step(s)   # 0 finishes its prompt (4 tokens, sampled), 1 gets the other 4
    assert [(e.id, e.start, len(e.tokens), e.sample) for e in plan.entries] == [(0, 16, 4, True), (1, 0, 4, False)]
    assert out[0][0] == 0
    plan, out = run_step(s)   # decode token of 0 beside the last prompt token of 1
    assert [(e.id, len(e.tokens), e.sample) for e in plan.entries] == [(0, 1, True), (1, 1, True)]
    assert plan.num_tokens == 2 and cache.check() == ""


def test_chunk_cap_and_two_token_portions():
    _, s = make(budget=64, chunk=2)
    s.add(0, list(range(7)), 2)
    sizes = []
    while s.has_unfinished():
        plan, _ = run_step(s)
        sizes.append([len(e.tokens) for e in plan.entries])
    assert sizes == [[2], [2], [2], [1], [1]]
    assert s.output(0) == [(0 * 31 + 7) % 97, (0 * 31 + 8) % 97]
    assert s.finish_reason(0) == H.FinishReason.LENGTH


def test_a_cap_on_portions_holds_further_prompts_back_but_not_single_tokens():
    cache = H.CacheManager([H.GroupSpec(4, 0)], [64], 4)
    s = H.Scheduler(cache, H.SchedulerConfig(4, 64, 64, 0, max_portions_per_step=1))
    s.add(0, list(range(9)), 6)
    s.add(1, list(range(7)), 6)
    s.add(2, [5], 6)            # a prompt of one token is no portion
    plan, _ = run_step(s)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(0, 9)]      # 1 waits, and 2 behind it (order of arrival)
    plan, _ = run_step(s)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 7), (2, 1)]
    plan, _ = run_step(s)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 1), (2, 1)]
    # a running request whose prompt is still being cut counts too, and later ones wait for it
    cache = H.CacheManager([H.GroupSpec(4, 0)], [64], 4)
    s = H.Scheduler(cache, H.SchedulerConfig(4, 8, 64, 0, max_portions_per_step=1))
    s.add(0, list(range(12)), 3)
    s.add(1, list(range(6)), 3)
    seen = []
    for _ in range(5):
        plan, _ = run_step(s)
        seen.append([(e.id, len(e.tokens)) for e in plan.entries])
        assert sum(len(e.tokens) > 1 for e in plan.entries) <= 1
    assert seen[:3] == [[(0, 8)], [(0, 4)], [(0, 1), (1, 6)]]
    with pytest.raises(Exception):
        H.Scheduler(cache, H.SchedulerConfig(4, 8, 64, 0, max_portions_per_step=-1))


def test_admission_is_fcfs_and_limited_by_seats():
    cache, s = make(seqs=2, slots=2, budget=64)
    for i in range(4):
        s.add(i, [1, 2, 3], 2)
    plan, _ = run_step(s)
    assert [e.id for e in plan.entries] == [0, 1] and s.num_waiting() == 2
    plan, _ = run_step(s)     # both produce their second token and finish
    assert s.is_finished(0) and s.is_finished(1)
    plan, _ = run_step(s)
    assert [e.id for e in plan.entries] == [2, 3]
    assert cache.check() == ""


def test_stop_token_finishes_and_is_not_kept():
    _, s = make()
    s.add(5, [9, 9], 10)
    toks = iter([11, 12, 77])
    reasons = []
    while s.has_unfinished():
        _, out = run_step(s, token_of=lambda rid, pos: next(toks), stop=77)
        reasons.append(out[0][2])
    assert s.output(5) == [11, 12] and reasons[-1] == H.FinishReason.STOP
    assert H.finish_reason_name(s.finish_reason(5)) == "stop"


def test_model_len_ends_a_request():
    _, s = make(model_len=8, budget=64)
    s.add(0, [1] * 5, 100)
    while s.has_unfinished():
        run_step(s)
    assert len(s.tokens(0)) == 8 and s.finish_reason(0) == H.FinishReason.MODEL_LEN


def test_bad_requests_are_refused_at_the_door():
    _, s = make(pages=4, page_size=4, model_len=64)
    with pytest.raises(ValueError, match="empty"):
        s.add(0, [], 4)
    with pytest.raises(ValueError, match="max_tokens"):
        s.add(0, [1], 0)
    with pytest.raises(ValueError, match="pages"):
        s.add(0, [1] * 16, 4)          # 17 tokens need 5 pages, the pool has 4
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(0, [1] * 64, 4)
    s.add(0, [1], 4)
    with pytest.raises(ValueError, match="in use"):
        s.add(0, [1], 4)


def test_out_of_pages_drops_the_latest_arrival_and_recomputes_it():
    cache, s = make(pages=8, page_size=4, budget=64)
    s.add(0, [1] * 7, 10)     # 2 pages, grows to 5
    s.add(1, [2] * 7, 10)
    s.add(2, [3] * 7, 10)
    plan, _ = run_step(s)     # all admitted (the third finds its 2 pages and one of growth for each of the others)
    assert len(plan.entries) == 3 and cache.free_pages(0) == 2
    plan, _ = run_step(s)     # token 8 of each fits its second page
    assert plan.preempted == []
    plan, _ = run_step(s)     # token 9 needs a third page each, two are left: 2 (the latest) is dropped, 0 and 1 go on
    assert plan.preempted == [2] and [e.id for e in plan.entries] == [0, 1]
    assert s.num_waiting() == 1 and s.preemptions_of(2) == 1 and s.preemptions_of(1) == 0
    assert cache.check() == "" and cache.live_requests() == 2 and cache.free_pages(0) == 2
    before = list(s.tokens(2))
    assert len(before) == 9   # its prompt and the two tokens it had produced
    came_back = None
    for _ in range(200):
        plan, _ = run_step(s)
        assert cache.check() == ""
        back = [e for e in plan.entries if e.id == 2]
        if back:
            came_back = back[0]
            break
    # it is recomputed as one prompt: its own prompt followed by what it had produced
    assert came_back is not None and came_back.start == 0 and came_back.sample
    assert list(came_back.tokens)[:9] == before
    while s.has_unfinished():
        run_step(s)
        assert cache.check() == ""
    for i in range(3):
        assert len(s.output(i)) == 10 and s.finish_reason(i) == H.FinishReason.LENGTH
        # no token was produced twice or lost: outputs follow the position rule
        assert s.output(i) == [(i * 31 + p) % 97 for p in range(7, 17)]
    assert s.stats().preemptions >= 1 and s.stats().recomputed_tokens > 0
    assert cache.free_pages(0) == 8 and cache.free_slots() == 4


def test_no_admission_in_a_step_that_preempted():
    cache, s = make(pages=5, page_size=4, budget=64, seqs=4)
    s.add(0, [1] * 8, 20)
    s.add(1, [2] * 7, 20)
    run_step(s)               # both admitted: 2 pages each, one left
    s.add(2, [3] * 2, 5)
    plan, _ = run_step(s)     # 0 takes the last page; 2 finds no room beside two running requests
    assert plan.preempted == [] and [e.id for e in plan.entries] == [0, 1] and s.num_waiting() == 1
    plan, _ = run_step(s)     # 1 needs a third page: it is the latest and is dropped; 2 must not slip in ahead of it
    assert plan.preempted == [1] and [e.id for e in plan.entries] == [0]
    assert s.num_waiting() == 2 and list(s.tokens(1))[:7] == [2] * 7


def test_admission_waits_for_room_for_the_whole_request():
    """Beside running requests a request is let in only when there are free pages for all its
    tokens and one page of growth for each running request; a request that was dropped waits
    the same way, so it is not read again just to be dropped again.  Alone, a request is let in
    on its first portion."""
    cache, s = make(pages=10, page_size=4, budget=8, seqs=4)
    s.add(0, [1] * 30, 4)     # alone: admitted on its first portion of 8 tokens
    plan, _ = run_step(s)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(0, 8)]
    s.add(1, [2] * 9, 4)      # 10 tokens = 3 pages, plus one for request 0: 4 <= 8 free pages
    s.add(2, [3] * 26, 4)     # 27 tokens = 7 pages, plus two: more than will be free while 0 and 1 run
    plan, _ = run_step(s)     # 0 continues (8 tokens): the budget is spent, nobody is admitted
    assert [e.id for e in plan.entries] == [0]
    for _ in range(3):
        plan, _ = run_step(s)
    # by now 0 has read its prompt (8 pages); 1 would need 3 + 1 pages: 2 are free
    assert s.num_running() == 1 and s.num_waiting() == 2 and s.stats().preemptions == 0
    while s.has_unfinished():
        run_step(s)
        assert cache.check() == ""
    assert s.stats().preemptions == 0 and all(len(s.output(i)) == 4 for i in range(3))
    assert cache.free_pages(0) == 10


def test_a_request_too_large_for_the_pool_ends_with_an_error():
    cache, s = make(pages=3, page_size=4, budget=64, model_len=64)
    s.add(0, [1] * 10, 30)    # fits at first (3 pages), cannot grow beyond 12 tokens
    reasons = []
    while s.has_unfinished():
        plan, out = run_step(s)
        reasons += [s.finish_reason(i) for i in plan.finished]
    assert reasons == [H.FinishReason.CACHE_EXHAUSTED]
    assert H.finish_reason_name(reasons[0]) == "kv_cache_exhausted"
    # 12 tokens fill the 3 pages; the 13th (the 3rd produced) can be sampled but not stored
    assert len(s.output(0)) == 3 and cache.free_pages(0) == 3 and cache.check() == ""


def test_random_workloads_finish_with_exact_token_counts():
    rng = random.Random(4)
    for trial in range(25):
        pages = rng.randint(6, 20)
        cache, s = make(pages=pages, page_size=4, slots=4, seqs=rng.randint(1, 4),
                        budget=rng.randint(2, 24), model_len=80, chunk=rng.choice([0, 0, 2, 5]))
        want = {}
        pending = []
        for i in range(rng.randint(3, 10)):
            n_prompt = rng.randint(1, min(4 * pages - 8, 30))
            n_out = rng.randint(1, max(1, min(20, 4 * pages - n_prompt - 1)))
            pending.append((i, [rng.randrange(97) for _ in range(n_prompt)], n_out))
            want[i] = n_out
        steps = 0
        while pending or s.has_unfinished():
            if pending and rng.random() < 0.5:
                s.add(*pending.pop(0))
            plan, _ = run_step(s)
            assert plan.num_tokens <= s.config().max_num_batched_tokens
            assert cache.check() == ""
            steps += 1
            assert steps < 5000, "the scheduler stopped making progress"
        for i, n in want.items():
            assert len(s.output(i)) == n and s.finish_reason(i) == H.FinishReason.LENGTH
        assert cache.free_pages(0) == pages and cache.free_slots() == 4


# ---- running one step ahead: tokens that are on the device but not yet known to the host

def run_ahead(sched, arrivals, token_of, stop, rng):
    """Drives the scheduler the way the engine does when it runs ahead: the next step is
    planned (with the placeholder in place of each token that was just sampled) before the
    values of the previous step's tokens are handed over."""
    in_flight = None          # sampled entries of the step whose tokens are not known yet
    steps = 0
    while arrivals or sched.has_unfinished() or in_flight is not None:
        if arrivals and rng.random() < 0.5:
            sched.add(*arrivals.pop(0))
        plan = sched.schedule()
        sched.commit(plan)
        for e in plan.entries:
            for t in e.tokens[:-1]:
                assert t != H.PENDING_TOKEN          # only the newest token may be unknown
        sched.mark_pending(plan)
        launched = [(e.id, e.start + len(e.tokens)) for e in plan.entries if e.sample]
        if in_flight is not None:
            for rid, pos in in_flight:
                if sched.is_live(rid):
                    tok = token_of(rid, pos)
                    sched.resolve(rid, tok, stop is not None and tok == stop)
        in_flight = launched or None
        steps += 1
        assert steps < 5000, "the scheduler stopped making progress"
    return steps


def test_running_ahead_gives_the_same_tokens():
    """Planning a step before the last step's tokens are known changes no request's output:
    with stop tokens, a token budget, chunked prompts and a pool so small that requests are
    dropped and recomputed, every request ends with the same tokens and the same reason as
    when every token is handed over at once."""
    token_of = lambda rid, pos: (rid * 31 + pos * 7) % 23
    for trial in range(40):
        rng = random.Random(100 + trial)
        pages = rng.randint(6, 20)
        kw = dict(pages=pages, page_size=4, slots=4, seqs=rng.randint(1, 4), budget=rng.randint(2, 24),
                  model_len=rng.choice([80, 24]), chunk=rng.choice([0, 0, 2, 5]))
        stop = rng.choice([None, 5, 11])
        reqs = []
        for i in range(rng.randint(3, 10)):
            n_prompt = rng.randint(1, min(4 * pages - 8, 20))
            n_out = rng.randint(1, max(1, min(20, 4 * pages - n_prompt - 1)))
            reqs.append((i, [rng.randrange(97) for _ in range(n_prompt)], n_out))
        # every token at once
        cache_a, a = make(**kw)
        arrivals, r2 = list(reqs), random.Random(trial)
        while arrivals or a.has_unfinished():
            if arrivals and r2.random() < 0.5:
                a.add(*arrivals.pop(0))
            run_step(a, token_of, stop)
        # one step ahead
        cache_b, b = make(**kw)
        run_ahead(b, list(reqs), token_of, stop, random.Random(trial))
        for i, _, _ in reqs:
            assert a.output(i) == b.output(i), (trial, i)
            assert a.finish_reason(i) == b.finish_reason(i), (trial, i)
            assert H.PENDING_TOKEN not in b.output(i)
        assert cache_b.check() == "" and cache_b.free_pages(0) == pages and cache_b.free_slots() == 4


def test_pending_token_protocol():
    cache, s = make(pages=8, budget=16)
    s.add(0, [1, 2, 3], 3)
    plan = s.schedule(); s.commit(plan); s.mark_pending(plan)
    assert s.has_pending(0) and s.output(0) == []            # the placeholder is not output
    plan2 = s.schedule(); s.commit(plan2)
    assert [(e.id, e.start, list(e.tokens), e.sample) for e in plan2.entries] == [(0, 3, [H.PENDING_TOKEN], True)]
    s.mark_pending(plan2)                                     # two on the way for a moment
    with pytest.raises(Exception):
        s.mark_pending(plan2)                                 # never three
    assert s.resolve(0, 42) == H.FinishReason.NONE and s.output(0) == [42]   # the older one first
    plan3 = s.schedule(); s.commit(plan3); s.mark_pending(plan3)             # its third token is the last by count
    assert s.resolve(0, 43) == H.FinishReason.NONE and s.output(0) == [42, 43]
    assert s.schedule().entries == []                         # nothing more to run for it
    assert s.has_unfinished()
    assert s.resolve(0, 44) == H.FinishReason.LENGTH and s.output(0) == [42, 43, 44]
    assert not s.has_unfinished() and cache.free_pages(0) == 8
    # a stop token drops what was sampled after it
    s.add(2, [7], 9)
    p1 = s.schedule(); s.commit(p1); s.mark_pending(p1)
    p2 = s.schedule(); s.commit(p2); s.mark_pending(p2)
    assert s.resolve(2, 5, True) == H.FinishReason.STOP and s.output(2) == []
    assert s.resolve(2, 6) == H.FinishReason.STOP            # the later value finds the request ended
    # a request that ends while its token is on the way drops that token
    s.add(1, [4, 5], 5)
    plan = s.schedule(); s.commit(plan); s.mark_pending(plan)
    s.abort(1)
    assert s.resolve(1, 9) == H.FinishReason.ABORTED and s.output(1) == []
    assert cache.check() == "" and cache.free_pages(0) == 8


def test_a_long_prompt_goes_through_a_small_windowed_pool_in_smaller_portions():
    """Only windowed layers (window 8, pages of 4), a pool of 6 pages = 24 tokens, a budget of
    64 tokens per step and a prompt of 100: one portion of 64 tokens would need 16 pages at once.
    The scheduler halves the portion until its pages fit, the window gives pages back after every
    step, and the request finishes with all its tokens instead of ending with an error."""
    cache = H.CacheManager([H.GroupSpec(4, 8)], [6], 2)
    s = H.Scheduler(cache, H.SchedulerConfig(2, 64, 256, 0))
    s.add(0, list(range(100)), 5)
    sizes = []
    steps = 0
    while s.has_unfinished():
        plan, _ = run_step(s)
        assert not plan.finished, "ended with an error although smaller portions fit"
        sizes.append([len(e.tokens) for e in plan.entries])
        assert cache.check() == ""
        steps += 1
        assert steps < 200
    assert s.finish_reason(0) == H.FinishReason.LENGTH and len(s.output(0)) == 5
    assert sum(n for step in sizes for n in step) == 100 + 4
    assert max(n for step in sizes for n in step) <= 16 and cache.free_pages(0) == 6
    # a pool that keeps every key gets no smaller portions: the request that is alone and
    # too large still ends at once (the prompt fits, its output does not)
    cache2, s2 = make(pages=3, page_size=4, budget=64)
    s2.add(0, list(range(11)), 8)
    reasons = []
    for _ in range(6):
        plan, _ = run_step(s2)
        reasons += [s2.finish_reason(i) for i in plan.finished]
    assert reasons == [H.FinishReason.CACHE_EXHAUSTED]

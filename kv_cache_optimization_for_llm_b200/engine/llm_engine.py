"""The engine: requests in, tokens out.

Each step asks the native scheduler for a plan (decode tokens of running requests
beside portions of prompts, under one token budget), runs it through the step
function and samples where a request reached the end of its known tokens.
Upstream's loop admits, runs a whole-prompt pass, then a decode pass, and waits for
the tokens before it goes on (base/src/main.cu:132-169); here one mixed pass does
both, and the engine runs one step ahead: the sampled tokens stay on the device, the
next step is planned and launched with placeholders that the embedding kernel
resolves there, and only then does the host wait for the step before it.  The GPU
so never idles while the host books tokens, plans and fills the next batch.  What a
stop token makes superfluous (one token of one request) is computed and dropped.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.paged_cache import host_runtime
from ..config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .runner import ModelRunner


@dataclass
class TokenEvent:
    """What one step did for one request."""
    request_id: int
    token: Optional[int]          # the new token, None when only a stop token ended it
    finished: bool
    reason: str = ""              # "stop", "length", "sequence_too_long", "kv_cache_exhausted"
    slot: int = -1


@dataclass
class _Live:
    params: SamplingParams
    key: int
    arrival_time: float
    first_token_time: Optional[float] = None
    in_slot: bool = False


@dataclass
class _InFlight:
    """A step that is on the device."""
    events: List[TokenEvent]            # what planning already decided (requests the cache can never hold)
    sampled: List[tuple]                # (request id, slot) per sampled row
    handle: object                      # the sampler's handle, None if nothing was sampled


class LLMEngine:
    def __init__(self, model_dir, config: Optional[EngineConfig] = None, random_init: Optional[dict] = None):
        self.config = config or EngineConfig()
        self.runner = ModelRunner(model_dir, self.config, random_init=random_init)
        host = host_runtime()
        self._host = host
        self.scheduler = host.Scheduler(self.runner.manager, host.SchedulerConfig(
            self.config.max_num_seqs, self.config.max_num_batched_tokens, self.runner.max_model_len,
            self.config.max_prefill_chunk, self.config.max_portions_per_step))
        self.sampler = Sampler(self.runner.vocab_size, self.config.max_num_seqs, self.runner.device,
                               self.config.seed, out=self.runner.sampled, status=self.runner.status)
        self._pending_token = int(host.PENDING_TOKEN)
        self._in_flight: Optional[_InFlight] = None
        self._row_of: Dict[int, int] = {}   # request -> its row in the last launch's sampling
        self.eos = set(self.runner.spec.eos_token_ids)
        self._live: Dict[int, _Live] = {}
        self._next_id = 0
        self.last_plan_tokens = 0

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None, key: Optional[int] = None) -> int:
        params = params or SamplingParams()
        if request_id is None:
            request_id = self._next_id
        self._next_id = max(self._next_id, request_id + 1)
        prompt = [int(t) for t in prompt]
        if any(t < 0 or t >= self.runner.vocab_size for t in prompt):
            raise ValueError(f"request {request_id}: a token id is outside the vocabulary of {self.runner.vocab_size}")
        self.scheduler.add(request_id, prompt, int(params.max_tokens))
        self._live[request_id] = _Live(params, request_id if key is None else int(key), time.perf_counter())
        return request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._in_flight is not None

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(request_id)
        self._live.pop(request_id, None)
        self._row_of.pop(request_id, None)

    def output(self, request_id: int) -> List[int]:
        return list(self.scheduler.output(request_id))

    def preemptions_of(self, request_id: int) -> int:
        return self.scheduler.preemptions_of(request_id)

    # ---------------------------------------------------------------- one step
    def _launch(self) -> Optional[_InFlight]:
        """Plans one step and puts it on the device: the step function, then the sampling
        kernel and the transfer of its tokens.  Waits for nothing.  None: nothing to run and
        nothing to report."""
        plan = self.scheduler.schedule()
        events: List[TokenEvent] = []
        for rid in plan.finished:   # ended because the cache can never hold them
            self._live.pop(rid, None)
            self._row_of.pop(rid, None)
            events.append(TokenEvent(rid, None, True, self._host.finish_reason_name(self.scheduler.finish_reason(rid))))
        for rid in plan.preempted:
            if rid in self._live:
                self._live[rid].in_slot = False
        self.last_plan_tokens = plan.num_tokens
        if not plan.entries:
            return _InFlight(events, [], None) if events else None
        manager = self.runner.manager
        entries, sampled = [], []
        for e in plan.entries:
            n = len(e.tokens)
            tokens = e.tokens
            if tokens[-1] == self._pending_token:
                # its newest token is still on the device: row of the last launch's sampling
                tokens = list(tokens)
                tokens[-1] = -(1 + self._row_of[e.id])
            entries.append(StepEntry(e.id, tokens, e.start, [n - 1] if e.sample else []))
            live = self._live[e.id]
            if not live.in_slot:
                # (Re)admitted: rebuild the slot's record of the tokens it produced.
                live.in_slot = True
                self.sampler.begin_request(manager.slot_of(e.id), live.params, self.scheduler.output(e.id))
            if e.sample:
                sampled.append(e)
        logits = self.runner.run(entries)
        self.scheduler.commit(plan)
        handle = None
        if sampled:
            handle = self.sampler.launch(
                logits, [self._live[e.id].params for e in sampled], [self._live[e.id].key for e in sampled],
                [e.start + len(e.tokens) for e in sampled], [manager.slot_of(e.id) for e in sampled])
            self.scheduler.mark_pending(plan)
            for row, e in enumerate(sampled):
                self._row_of[e.id] = row
        return _InFlight(events, [(e.id, manager.slot_of(e.id)) for e in sampled], handle)

    def _complete(self, flight: _InFlight) -> List[TokenEvent]:
        """Waits for a launched step's tokens and books them."""
        events = flight.events
        if flight.handle is None:
            return events
        toks, status = self.sampler.read(flight.handle)
        self.runner.check_status(status)
        for (rid, slot), tok in zip(flight.sampled, toks):
            live = self._live.get(rid)
            if live is None:
                continue        # ended meanwhile (a stop token one step earlier, an abort): computed for nothing
            is_stop = (tok in self.eos) and not live.params.ignore_eos
            reason = self.scheduler.resolve(rid, int(tok), is_stop)
            finished = reason != self._host.FinishReason.NONE
            if live.first_token_time is None:
                live.first_token_time = time.perf_counter()
            events.append(TokenEvent(rid, None if is_stop else int(tok), finished,
                                     self._host.finish_reason_name(reason) if finished else "", slot))
            if finished:
                self._live.pop(rid, None)
                self._row_of.pop(rid, None)
        return events

    def step(self) -> List[TokenEvent]:
        """Returns what one step did.  With ``run_ahead`` the step after it is already on the
        device when this one's tokens are waited for."""
        flight = self._in_flight if self._in_flight is not None else self._launch()
        self._in_flight = None
        if flight is None:
            return []
        if self.config.run_ahead and flight.handle is not None:
            self._in_flight = self._launch()
        return self._complete(flight)

    # ---------------------------------------------------------------- convenience
    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[List[int]]:
        """Runs the prompts to completion and returns each one's new tokens."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_unfinished():
            self.step()
        return [list(self.scheduler.take_finished(i)) for i in ids]

    def stats(self) -> dict:
        s = self.scheduler.stats()
        m = self.runner.manager
        return {"steps": s.steps, "scheduled_tokens": s.scheduled_tokens, "preemptions": s.preemptions,
                "recomputed_tokens": s.recomputed_tokens, "finished": s.finished,
                "running": self.scheduler.num_running(), "waiting": self.scheduler.num_waiting(),
                "free_pages": [m.free_pages(g) for g in range(m.num_groups())],
                "num_pages": [m.num_pages(g) for g in range(m.num_groups())],
                "step_kinds": dict(self.runner.step_kinds)}

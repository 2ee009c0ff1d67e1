"""Continuous batching: which requests run which tokens in the next step.

The reference's only scheduler is the loop of ``bench continuous``
(apps/cli/main.cpp:1451-1644): every live slot contributes its one decode
row, and at most one waiting request is admitted per step with its whole
prompt.  This scheduler keeps that shape (decodes first, then prompt work)
and adds what a paged cache needs:

* admission in arrival order while a state slot is free, fewer than
  ``max_requests`` run, and the pages of the first portion are free;
* a token budget per step (``max_batch_tokens``): running requests take their
  next tokens first (one for a decoding request, a portion of at most
  ``chunk`` tokens for one still in its prompt), new requests fill what is left;
* finishing on ``max_new_tokens``, on an end token, or at the context limit
  (src/apps: main.cpp:1587-1592), freeing pages and slot in the same step;
* when pages run out for a running request, the most recently admitted
  running request is preempted: everything it holds is freed and it goes back
  to the head of the queue, to be recomputed later from its prompt plus what
  it generated so far (its sampler state travels with it, so its output does
  not change).  No new request is admitted in a step that preempted.  A
  request that could not fit the empty pool is refused when it is submitted.

Decisions depend only on the queue and the pools, never on time, so a run can
be replayed.  The scheduler needs no GPU: it talks to the cache manager and
hands out plans; whoever runs them reports the sampled tokens back through
:meth:`update`.

The queues, the planning and the bookkeeping are C++ (csrc/runtime.cpp:
``TgeRtScheduler``), which also keeps each request's tokens so that a plan can
be packed into the step's index arrays without passing through Python lists.
:class:`Request` here carries what the sampler needs (parameters, generator
state, the tokens generated so far) and mirrors the rest.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from .. import runtime as _rt
from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams, XorShift32
from .batch import Portion

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
_STATES = (WAITING, RUNNING, FINISHED)
_REASONS = ("end_token", "length", "context")


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    rng: XorShift32 = field(default_factory=XorShift32)
    _scheduler: Optional["Scheduler"] = field(default=None, repr=False, compare=False)
    _last: tuple = field(default=(WAITING, 0, 0), repr=False, compare=False)   # state, computed, preemptions at finish

    def __post_init__(self) -> None:
        self.rng = XorShift32(self.sampling.seed)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def _info(self) -> tuple:
        if self._scheduler is None:
            return self._last
        return self._scheduler._info(self.id)

    @property
    def state(self) -> str:
        return self._info()[0]

    @property
    def computed(self) -> int:
        """Tokens whose cache entries exist."""
        return self._info()[1]

    @property
    def preemptions(self) -> int:
        return self._info()[2]

    def token_slice(self, start: int, count: int) -> List[int]:
        """Tokens [start, start + count) of prompt-then-output, without building the whole list."""
        split = len(self.prompt)
        if start >= split:
            return self.output[start - split:start - split + count]
        if start + count <= split:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - split]


@dataclass
class ScheduledPortion:
    request: Request
    start: int
    count: int
    samples: bool          # the portion ends at the request's last known token: a new token is drawn


@dataclass
class StepPlan:
    items: List[ScheduledPortion] = field(default_factory=list)
    preempted: List[Hashable] = field(default_factory=list)
    scheduler: Optional["Scheduler"] = field(default=None, repr=False)

    @property
    def num_tokens(self) -> int:
        return sum(item.count for item in self.items)

    def portions(self) -> List[Portion]:
        out = []
        for item in self.items:
            tokens = item.request.token_slice(item.start, item.count)
            out.append(Portion(item.request.id, tokens, [item.count - 1] if item.samples else []))
        return out

    def pack(self, vocab_size: int, fixed_width: int, pad_rows: int, out: np.ndarray, layout: "_rt.StepLayout") -> int:
        """Packs the plan's index arrays into ``out`` (int32) straight from the runtime's own token copies."""
        s = self.scheduler
        return _rt.check(s._lib.tge_rt_sched_pack(s._native, int(vocab_size), int(fixed_width), int(pad_rows),
                                                  out.ctypes.data, out.size, ctypes.byref(layout)))


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_tokens: int, max_requests: int, max_model_len: int,
                 chunk: Optional[int] = None, end_token_ids: Sequence[int] = ()):
        if max_batch_tokens <= 0 or max_requests <= 0 or max_model_len <= 0:
            raise ValueError("scheduler: limits must be positive")
        if chunk is not None and chunk <= 0:
            raise ValueError("scheduler: chunk must be positive")
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_requests = min(max_requests, cache.max_requests)
        self.max_model_len = max_model_len
        self.chunk = chunk
        self.end_token_ids = frozenset(int(t) for t in end_token_ids)
        self._lib = _rt.lib()
        ends = (ctypes.c_int * max(len(self.end_token_ids), 1))(*sorted(self.end_token_ids))
        self._native = self._lib.tge_rt_sched_create(cache.native, int(max_batch_tokens), int(max_requests),
                                                     int(max_model_len), int(chunk or 0), ends, len(self.end_token_ids))
        if not self._native:
            _rt.check(_rt.VALUE_ERROR)
        self._requests: Dict[Hashable, Request] = {}          # waiting or running
        self.finished: Dict[Hashable, Request] = {}
        most = max(self.max_requests, 1)
        self._ids = (ctypes.c_int64 * most)()
        self._starts = (ctypes.c_int * most)()
        self._counts = (ctypes.c_int * most)()
        self._samples = (ctypes.c_int * most)()
        self._reasons = (ctypes.c_int * most)()

    def __del__(self):
        if getattr(self, "_native", None):
            self._lib.tge_rt_sched_destroy(self._native)
            self._native = None

    # -- views ----------------------------------------------------------------
    def _info(self, request: Hashable) -> tuple:
        state, computed, preemptions, tokens = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        _rt.check(self._lib.tge_rt_sched_request_info(self._native, self.cache.handle_of(request), ctypes.byref(state),
                                                      ctypes.byref(computed), ctypes.byref(preemptions),
                                                      ctypes.byref(tokens)))
        return _STATES[state.value], computed.value, preemptions.value

    def _listed(self, function) -> List[Request]:
        count = function(self._native, self._ids, len(self._ids))
        if count > len(self._ids):
            self._ids = (ctypes.c_int64 * count)()
            count = function(self._native, self._ids, count)
        return [self._requests[self.cache.name_of(h)] for h in self._ids[:count]]

    @property
    def waiting(self) -> List[Request]:
        return self._listed(self._lib.tge_rt_sched_waiting)

    @property
    def running(self) -> List[Request]:
        return self._listed(self._lib.tge_rt_sched_running)

    @property
    def counters(self) -> Dict[str, int]:
        names = ("steps", "tokens", "preemptions", "admitted", "finished")
        return {name: int(self._lib.tge_rt_sched_counter(self._native, i)) for i, name in enumerate(names)}

    # -- submission -----------------------------------------------------------
    def add(self, request: Request) -> None:
        request.sampling.validate()
        if request.id in self._requests:
            raise ValueError(f"request id {request.id!r} is already in use")
        prompt = np.ascontiguousarray(request.prompt, dtype=np.int32)
        known = request.id in self.cache._handles
        handle = self.cache.pin(request.id)
        try:
            _rt.check(self._lib.tge_rt_sched_add(self._native, handle, prompt.ctypes.data, int(prompt.size),
                                                 int(request.max_new_tokens)))
        except Exception:
            if not known:
                self.cache.unpin(request.id)
            raise
        request._scheduler = self
        self._requests[request.id] = request
        self.finished.pop(request.id, None)

    def num_waiting(self) -> int:
        return int(self._lib.tge_rt_sched_waiting(self._native, self._ids, 0))

    def has_work(self) -> bool:
        return bool(self._lib.tge_rt_sched_has_work(self._native))

    # -- one step's plan ------------------------------------------------------
    def schedule(self) -> StepPlan:
        count = self._lib.tge_rt_sched_schedule(self._native)
        if count < 0:
            _rt.check(count)
        if count > len(self._starts):
            self._ids = (ctypes.c_int64 * count)()
            self._starts, self._counts = (ctypes.c_int * count)(), (ctypes.c_int * count)()
            self._samples, self._reasons = (ctypes.c_int * count)(), (ctypes.c_int * count)()
        self._lib.tge_rt_sched_plan(self._native, self._ids, self._starts, self._counts, self._samples, count)
        name_of, requests = self.cache._names, self._requests
        plan = StepPlan(scheduler=self)
        plan.items = [ScheduledPortion(requests[name_of[self._ids[i]]], self._starts[i], self._counts[i],
                                       bool(self._samples[i])) for i in range(count)]
        preempted = self._lib.tge_rt_sched_plan_preempted(self._native, self._ids, len(self._ids))
        if preempted:
            plan.preempted = [name_of[h] for h in self._ids[:min(preempted, len(self._ids))]]
        if self.cache.state_storage:
            for item in plan.items:           # a request that starts (over) gets a zeroed state slot
                if item.start == 0:
                    self.cache.zero_state(self.cache.slot_of(item.request.id))
        return plan

    # -- after the step -------------------------------------------------------
    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Records the step: ``sampled`` holds one token per sampling portion, in plan order."""
        tokens = np.ascontiguousarray(sampled, dtype=np.int32)
        cursor = 0
        for item in plan.items:
            if item.samples and cursor < tokens.size:
                item.request.output.append(int(tokens[cursor]))
                cursor += 1
        try:
            done = _rt.check(self._lib.tge_rt_sched_update(self._native, tokens.ctypes.data, int(tokens.size), self._ids,
                                                           self._reasons, min(len(self._ids), len(self._reasons))))
        except Exception:
            cursor = 0
            for item in plan.items:           # the step was not recorded: take the tokens back
                if item.samples and cursor < tokens.size:
                    item.request.output.pop()
                    cursor += 1
            raise
        finished: List[Request] = []
        for i in range(done):
            request = self._requests.pop(self.cache.name_of(self._ids[i]))
            request.finish_reason = _REASONS[self._reasons[i]]
            request._last = (FINISHED,) + self._info(request.id)[1:]
            request._scheduler = None
            self._lib.tge_rt_sched_forget(self._native, self.cache.handle_of(request.id))
            self.cache.unpin(request.id)
            self.finished[request.id] = request
            finished.append(request)
        return finished

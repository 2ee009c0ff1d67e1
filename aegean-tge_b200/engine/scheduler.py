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
hands out :class:`Portion` lists; whoever runs them reports the sampled
tokens back through :meth:`update`.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams, XorShift32
from .batch import Portion

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingParams = field(default_factory=SamplingParams)
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    computed: int = 0                 # tokens whose cache entries exist
    finish_reason: Optional[str] = None
    preemptions: int = 0
    rng: XorShift32 = field(default_factory=XorShift32)

    def __post_init__(self) -> None:
        self.rng = XorShift32(self.sampling.seed)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

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

    @property
    def num_tokens(self) -> int:
        return sum(item.count for item in self.items)

    def portions(self) -> List[Portion]:
        out = []
        for item in self.items:
            tokens = item.request.token_slice(item.start, item.count)
            out.append(Portion(item.request.id, tokens, [item.count - 1] if item.samples else []))
        return out


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
        self.end_token_ids = frozenset(end_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order
        self.finished: Dict[Hashable, Request] = {}
        self.counters = {"steps": 0, "tokens": 0, "preemptions": 0, "admitted": 0, "finished": 0}

    # -- submission -----------------------------------------------------------
    def add(self, request: Request) -> None:
        request.sampling.validate()
        if not request.prompt:
            raise ValueError(f"request {request.id!r}: at least one prompt token is required")
        if request.max_new_tokens <= 0:
            raise ValueError(f"request {request.id!r}: max_new_tokens must be positive")
        if len(request.prompt) + 1 > self.max_model_len:
            raise ValueError(f"request {request.id!r}: {len(request.prompt)} prompt tokens leave no room in a "
                             f"context of {self.max_model_len}")
        # the last generated token is never fed back, so a request caches at most prompt + new - 1 tokens
        most = min(len(request.prompt) + request.max_new_tokens - 1, self.max_model_len)
        if not self.cache.fits_empty_pool(most):
            raise ValueError(f"request {request.id!r}: {most} tokens do not fit the page pool even when it is empty")
        if any(r.id == request.id for r in self.waiting) or any(r.id == request.id for r in self.running):
            raise ValueError(f"request id {request.id!r} is already in use")
        request.state = WAITING
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step's plan ------------------------------------------------------
    def _portion_size(self, request: Request, budget: int) -> int:
        remaining = request.num_tokens - request.computed
        count = min(remaining, budget)
        if self.chunk is not None:
            count = min(count, self.chunk)
        return count

    def _preempt(self, request: Request, plan: StepPlan) -> None:
        self.cache.free(request.id)
        self.running.remove(request)
        request.state = WAITING
        request.computed = 0
        request.preemptions += 1
        self.waiting.appendleft(request)
        plan.preempted.append(request.id)
        plan.items = [item for item in plan.items if item.request is not request]
        self.counters["preemptions"] += 1

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_batch_tokens
        # running requests first, in admission order; each reserves its pages as it is planned
        index = 0
        while index < len(self.running):
            request = self.running[index]
            count = self._portion_size(request, budget)
            if count <= 0:
                index += 1
                continue
            while not self.cache.can_grow(request.id, request.computed + count):
                victim = self.running[-1]
                self._preempt(victim, plan)
                # give the victim's planned tokens back to the budget
                budget = self.max_batch_tokens - plan.num_tokens
                if victim is request:
                    break
            if request.state != RUNNING:
                continue                      # it preempted itself; the list is one shorter, same index
            count = self._portion_size(request, budget)
            self.cache.grow(request.id, request.computed + count)
            plan.items.append(ScheduledPortion(request, request.computed, count,
                                               request.computed + count == request.num_tokens))
            budget -= count
            index += 1
        # then new requests, in arrival order, unless this step had to preempt
        # (or unless preemption left nothing to run: then the head of the queue starts over at once)
        while (self.waiting and (not plan.preempted or not plan.items) and budget > 0
               and len(self.running) < self.max_requests and self.cache.free_slots > 0):
            request = self.waiting[0]
            count = self._portion_size(request, budget)
            pages = -(-count // self.cache.page_size)
            if any(pages > group.pool.free_count for group in self.cache.groups):
                break
            self.waiting.popleft()
            self.cache.admit(request.id)
            self.cache.grow(request.id, count)
            request.state = RUNNING
            request.computed = 0
            self.running.append(request)
            self.counters["admitted"] += 1
            plan.items.append(ScheduledPortion(request, 0, count, count == request.num_tokens))
            budget -= count
        if not plan.items and self.has_work():
            raise RuntimeError("scheduler: nothing can run although requests are waiting "
                               "(the page pool is too small for the oldest request's next portion)")
        self.counters["steps"] += 1
        self.counters["tokens"] += plan.num_tokens
        return plan

    # -- after the step -------------------------------------------------------
    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Records the step: ``sampled`` holds one token per sampling portion, in plan order."""
        finished: List[Request] = []
        cursor = 0
        for item in plan.items:
            request = item.request
            request.computed = item.start + item.count
            self.cache.set_computed(request.id, request.computed)
            if not item.samples:
                continue
            token = int(sampled[cursor])
            cursor += 1
            request.output.append(token)
            reason = None
            if token in self.end_token_ids:
                reason = "end_token"
            elif len(request.output) >= request.max_new_tokens:
                reason = "length"
            elif request.num_tokens >= self.max_model_len:
                reason = "context"
            if reason is not None:
                request.state = FINISHED
                request.finish_reason = reason
                self.cache.free(request.id)
                self.running.remove(request)
                self.finished[request.id] = request
                finished.append(request)
                self.counters["finished"] += 1
        if cursor != len(sampled):
            raise ValueError(f"scheduler: {len(sampled)} sampled tokens for {cursor} sampling portions")
        return finished

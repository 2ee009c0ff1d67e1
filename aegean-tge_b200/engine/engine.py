"""The Python entry point: load a model folder, generate tokens.

    engine = Engine("path/to/model", dtype="bfloat16")
    ids = engine.generate([5, 17, 3], n=32)                      # greedy
    ids = engine.generate([[1, 2], [3]], n=8, sampling=SamplingParams(temperature=0.8, seed=7))

Options carry the reference's names and meanings where it has them
(``generate --model --tokens --n --temp --top-k --top-p --min-p
--repeat-penalty --penalty-window --seed --context``, apps/cli/main.cpp:84-120):
``context`` caps the cached length (default 4096, capped by the model,
src/models/qwen2.cpp:424-430), ``n`` is the number of tokens to generate,
sampling fields are those of :class:`SamplingParams`.  What is new here
(pages, token budget, chunk) has no counterpart there.

An engine owns one model, one cache manager, one step function, one
scheduler and one sampler; ``bin/trace_run`` and the benchmarks drive the
same objects.
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, Hashable, List, Optional, Sequence, Union

import torch

from .. import ops as _ops
from .. import runtime as _rt
from ..cache.manager import CacheManager
from ..config.common import ConfigError, read_config_json
from ..models.decoder import DecoderModel
from ..parts.base import BuildEnv
from ..registry import architecture_of
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_checkpoint
from ..weights.random_init import fill_random, parse_dtype
from .batch import Portion
from .runner import ModelRunner
from .scheduler import Request, Scheduler

DEFAULT_CONTEXT = 4096      # the reference's default KV length (src/models/qwen2.cpp:25)
# Tokens per page.  The reference's unwired block table uses 16 (kBlockTokens, block_table.hpp:19), and 16 is
# fully supported (``page_size=16``).  The default is 64, one attention tile: the kernels fetch K and V by TMA
# one box per page and 64 columns, and an SM's TMA unit moves 2 KB boxes (16-token pages) at about 18 bytes per
# clock but 8 KB boxes (64-token pages) at about 31, which is what long contexts are read at.
PAGE_SIZE = 64


class Engine:
    def __init__(self, model_dir: Optional[str] = None, *, dtype: str = "bfloat16", context: Optional[int] = None,
                 max_tokens: Optional[int] = None, num_pages: Optional[int] = None, max_batch_tokens: int = 2048,
                 max_requests: int = 64, chunk: Optional[int] = None, device: str = "cuda:0",
                 memory_fraction: float = 0.9, random_config: Optional[Dict[str, Any]] = None, seed: int = 0,
                 page_size: int = PAGE_SIZE, run_ahead: bool = True, use_graphs: bool = True):
        """``model_dir``: folder with config.json and model.safetensors.  Alternatively
        ``random_config`` (a config.json as a dict) and ``seed``: random weights drawn on the device.

        Cache size, first match wins: ``num_pages`` pages per group; ``max_tokens`` cached
        tokens in total; else ``memory_fraction`` of the memory left after the weights.
        ``run_ahead`` / ``use_graphs``: switches for the step queued ahead and for CUDA graph replay of
        single-token steps (both on; off for A/B comparisons).
        """
        if not torch.cuda.is_available():
            raise RuntimeError("this engine runs on a CUDA device only; none is available")
        if (model_dir is None) == (random_config is None):
            raise ValueError("give either model_dir or random_config")
        if page_size <= 0 or 64 % page_size != 0:
            raise ValueError(f"page_size {page_size} must divide 64, the attention kernels' tile of key positions")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        raw = read_config_json(model_dir) if model_dir is not None else dict(random_config)
        self.raw_config = raw
        self.architecture = architecture_of(raw)
        self.config = self.architecture.parse_config(raw)
        self.spec = self.architecture.build_spec(self.config)
        limit = DEFAULT_CONTEXT if context is None else int(context)
        if limit <= 0:
            raise ValueError("context must be positive")
        self.max_model_len = min(self.spec.max_positions, limit)
        started = time.time()
        env = BuildEnv(dtype=self.dtype, device=self.device, hidden_size=self.spec.hidden_size,
                       max_positions=self.max_model_len, page_size=page_size, ops=_ops)
        _ops.core()     # builds and loads the kernels now, or fails loudly
        self.model = DecoderModel(self.spec, env)
        if model_dir is not None:
            load_checkpoint(self.model, model_dir)
        else:
            fill_random(self.model, raw, seed)
        self.load_seconds = time.time() - started
        self.cache = CacheManager(page_size, max_requests)
        self.model.declare_cache(self.cache)
        element = 2 if self.dtype == torch.bfloat16 else 4
        if num_pages is not None:
            sizes = [int(num_pages)] * len(self.cache.groups)
        elif max_tokens is not None:
            sizes = self.cache.plan_pool_sizes(tokens=int(max_tokens))
        else:
            torch.cuda.synchronize(self.device)
            free, _total = torch.cuda.mem_get_info(self.device)
            reserve = 2 << 30     # activations of a full step, logits, scratch
            budget = max(int(free * memory_fraction) - reserve, 0)
            sizes = self.cache.plan_pool_sizes(budget_bytes=budget, element_size=element)
            most = max_requests * -(-self.max_model_len // page_size)
            sizes = [min(s, most) for s in sizes]
        self.cache.set_pool_sizes(sizes)
        self.cache.allocate_storage(self.dtype, self.device)
        self.model.attach_cache(self.cache)
        self.runner = ModelRunner(self.model, self.cache, self.max_model_len, use_graphs=use_graphs)
        self.scheduler = Scheduler(self.cache, max_batch_tokens=max_batch_tokens, max_requests=max_requests,
                                   max_model_len=self.max_model_len, chunk=chunk,
                                   end_token_ids=self.spec.end_token_ids)
        self.sampler = Sampler(_ops, self.device)
        self._next_id = 0
        self.d2h_bytes_last = 0
        self.run_ahead = run_ahead
        self._ahead = None
        self.ahead_used = 0
        self.ahead_dropped = 0

    # -- requests -------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], n: int = 32, sampling: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        """Queues a request for ``n`` new tokens; returns its id."""
        for token in prompt:
            if not 0 <= int(token) < self.spec.vocab_size:
                raise ValueError(f"token {token} is outside the vocabulary")
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        self.scheduler.add(Request(request_id, [int(t) for t in prompt], int(n), sampling or SamplingParams()))
        return request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> List[Request]:
        """Plans one step, runs it, samples, and returns the requests that finished in it.

        While every live request is decoding with a sampler that stays on the device, the next step is
        queued before this step's tokens are read (its token ids are taken from the device), so the GPU
        does not wait for the host between steps.  The step queued ahead is used only if the scheduler
        then plans exactly that step; otherwise (a request ended on an end token, a new one arrived, pages
        ran out) its results are dropped, the generators it drew from are put back, and the planned step
        runs as usual.  What it wrote into the pages lies beyond every request's recorded length; fixed-size
        state that mixers update in place is copied before the step ahead runs and put back when it is dropped.
        """
        plan = self.scheduler.schedule()
        ahead, self._ahead = self._ahead, None
        pending = None
        if ahead is not None:
            if self._matches(ahead, plan):
                pending = ahead["result"]
                self.ahead_used += 1
            else:
                for request, state in zip(ahead["requests"], ahead["rng_states"]):
                    request.rng.state = state
                self.cache.restore_state(ahead["state"])
                self.ahead_dropped += 1
        sampling_items = [item for item in plan.items if item.samples]
        if pending is None:
            logits = self.runner.step_plan(plan)
            if sampling_items:
                params = [item.request.sampling for item in sampling_items]
                if self.run_ahead and Sampler.stays_on_device(params):
                    pending = self.sampler.sample_async(logits, params, [item.request.rng for item in sampling_items])
                else:
                    sampled = self.sampler.sample(logits, params, [item.request.rng for item in sampling_items],
                                                  [item.request.tokens if item.request.sampling.has_penalty else ()
                                                   for item in sampling_items])
                    self.d2h_bytes_last = 4 * len(sampled)
                    return self.scheduler.update(plan, sampled)
            else:
                return self.scheduler.update(plan, [])
        ids, host, event = pending
        if self._may_run_ahead(plan):
            self._ahead = self._launch_ahead(plan, ids)
        event.synchronize()
        sampled = host.tolist()
        self.d2h_bytes_last = 4 * len(sampled)
        return self.scheduler.update(plan, sampled)

    # -- the step queued ahead ----------------------------------------------------
    def _may_run_ahead(self, plan) -> bool:
        items = plan.items
        if not self.run_ahead or not items or not self.runner.can_step_ahead(len(items)):
            return False
        if self.scheduler.num_waiting():
            return False
        for item in items:
            request = item.request
            if item.count != 1 or not item.samples:
                return False
            # the token this step draws must not be the request's last, and must leave room for one more
            if len(request.output) + 1 >= request.max_new_tokens or request.num_tokens + 2 > self.max_model_len:
                return False
        return Sampler.stays_on_device([item.request.sampling for item in items])

    def _launch_ahead(self, plan, ids: torch.Tensor):
        """Queues the step after ``plan`` for the same requests, fed with ``ids`` from the device."""
        from ..cache.pages import PoolExhausted
        requests = [item.request for item in plan.items]
        names = [r.id for r in requests]
        # this step's tokens are computed as far as the cache is concerned (the scheduler records the same later)
        for item in plan.items:
            self.cache.set_computed(item.request.id, item.start + item.count)
        states = [r.rng.state for r in requests]
        snapshot = (self.cache.snapshot_state([self.cache.slot_of(name) for name in names])
                    if self.cache.state_storage else None)
        try:
            logits = self.runner.step_ahead(names, ids)
        except PoolExhausted:
            return None
        result = self.sampler.sample_async(logits, [r.sampling for r in requests], [r.rng for r in requests])
        return {"requests": requests, "starts": [item.start + 1 for item in plan.items], "rng_states": states,
                "state": snapshot, "result": result}

    @staticmethod
    def _matches(ahead, plan) -> bool:
        items = plan.items
        if len(items) != len(ahead["requests"]):
            return False
        for item, request, start in zip(items, ahead["requests"], ahead["starts"]):
            if item.request is not request or item.start != start or item.count != 1 or not item.samples:
                return False
        return True

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], n: int = 32,
                 sampling: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> Union[List[int], List[List[int]]]:
        """Generates ``n`` tokens for one prompt (a list of ids) or several (a list of lists)."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        batch = [prompts] if single else list(prompts)
        if isinstance(sampling, SamplingParams) or sampling is None:
            params = [sampling] * len(batch)
        else:
            params = list(sampling)
            if len(params) != len(batch):
                raise ValueError("one SamplingParams per prompt")
        ids = [self.add_request(p, n, s) for p, s in zip(batch, params)]
        done: Dict[Hashable, Request] = {}
        while len(done) < len(ids):
            for request in self.step():
                done[request.id] = request
        _ops.check_status()
        outputs = [done[i].output for i in ids]
        for i in ids:
            self.scheduler.finished.pop(i, None)
        return outputs[0] if single else outputs

    # -- facts ----------------------------------------------------------------
    def stats(self) -> Dict[str, Any]:
        out = dict(self.scheduler.counters)
        out["pages"] = [{"capacity": g.pool.capacity, "free": g.pool.free_count, "layers": len(g.layers),
                         "window": g.spec.window} for g in self.cache.groups]
        out["steps_queued_ahead"] = {"used": self.ahead_used, "dropped": self.ahead_dropped}
        out["runner_steps"] = self.runner.steps
        out["runner_tokens"] = self.runner.tokens_run
        out["libraries"] = list(_ops.loaded_libraries()) + [_rt.library_path()]
        return out

    def describe(self) -> Dict[str, Any]:
        kinds: Dict[str, int] = {}
        for layer in self.spec.layers:
            name = f"{layer.mixer.kind}+{layer.feed_forward.kind}"
            kinds[name] = kinds.get(name, 0) + 1
        return {
            "layer_kinds": ", ".join(f"{count} x {name}" for name, count in kinds.items()),
            "architecture": self.spec.architecture, "dtype": str(self.dtype).replace("torch.", ""),
            "layers": len(self.spec.layers), "hidden_size": self.spec.hidden_size, "vocab_size": self.spec.vocab_size,
            "max_model_len": self.max_model_len, "page_size": self.cache.page_size,
            "pages_per_group": [g.pool.capacity for g in self.cache.groups],
            "param_bytes_per_step": self.model.step_param_bytes(),
            "cache_bytes_per_token": self.model.cache_bytes_per_token(),
            "load_seconds": round(self.load_seconds, 3),
        }

"""The step function: a batch of portions in, logits at the wanted places out.

``ModelRunner.step`` runs exactly the tokens it is given, as one batch,
against what earlier steps left in the cache: it grows each request's pages,
describes the batch to the kernels, runs the model once and returns float32
logits for the wanted rows, in the order of the portions and of their
``want`` lists.  It samples nothing and schedules nothing.  The reference's
counterpart is ``Qwen2::forward_batch`` (src/models/qwen2.cpp:1613-1946),
which stores all rows' K/V and then lets every row attend up to its own
position, so that prompt rows of one request and decode rows of others share
one weight pass.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..cache.pages import PoolExhausted
from ..models.decoder import DecoderModel
from .batch import Portion, build_context


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_model_len: int):
        self.model = model
        self.cache = cache
        self.max_model_len = max_model_len
        self.device = model.env.device
        self.ops = model.env.ops
        self.steps = 0
        self.tokens_run = 0
        self.h2d_bytes_last = 0

    # -- request lifetime -----------------------------------------------------
    def is_live(self, request: Hashable) -> bool:
        return self.cache.is_live(request)

    def computed(self, request: Hashable) -> int:
        return self.cache.computed(request)

    def finish(self, request: Hashable) -> None:
        """Gives back the request's pages and slot."""
        self.cache.free(request)

    # -- the step -------------------------------------------------------------
    def step(self, portions: Sequence[Portion]) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns float32 logits [wanted rows, vocab] on the device, or None."""
        if not portions:
            return None
        seen = set()
        vocab = self.model.spec.vocab_size
        for portion in portions:
            if portion.request in seen:
                raise ValueError(f"request {portion.request!r} appears twice in one step")
            seen.add(portion.request)
            portion.validate(vocab)
        # reserve everything before touching anything, so a step either runs whole or not at all
        # (a request the scheduler already admitted and grew is left as it is: both calls are idempotent)
        admitted: List[Hashable] = []
        try:
            for portion in portions:
                if not self.cache.is_live(portion.request):
                    self.cache.admit(portion.request)
                    admitted.append(portion.request)
                total = self.cache.computed(portion.request) + len(portion.tokens)
                if total > self.max_model_len:
                    raise ValueError(f"request {portion.request!r}: {total} tokens exceed the context of {self.max_model_len}")
                self.cache.grow(portion.request, total)
        except (PoolExhausted, ValueError):
            for request in admitted:
                self.cache.free(request)
            raise
        requests = [p.request for p in portions]
        starts = [self.cache.computed(r) for r in requests]
        slots = [self.cache.slot_of(r) for r in requests]
        tables = [self.cache.block_table(g, requests) for g in range(len(self.cache.groups))]
        ctx, rows, h2d = build_context(portions, starts, slots, tables, self.device)
        self.h2d_bytes_last = h2d
        logits = self.model.forward(ctx, rows)
        for portion, start in zip(portions, starts):
            self.cache.set_computed(portion.request, start + len(portion.tokens))
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        return logits

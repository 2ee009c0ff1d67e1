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
    def __init__(self, model: DecoderModel, cache: CacheManager, max_model_len: int, use_graphs: bool = True,
                 max_graph_batch: int = 256):
        """``use_graphs``: steps made only of single tokens replay a CUDA graph captured per batch size."""
        self.use_graphs = use_graphs and model.graph_safe      # a part that works from host values runs eagerly
        self.max_graph_batch = max_graph_batch
        self._graphs: Dict[tuple, "DecodeGraph"] = {}
        self.graph_replays = 0
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
        batch = len(portions)
        if self.use_graphs and batch <= self.max_graph_batch and all(len(p.tokens) == 1 for p in portions):
            bound = 1024
            while bound < max(starts) + 1:
                bound *= 2
            bound = min(bound, self.max_model_len)
            graph = self._graphs.get((batch, bound))
            if graph is None:
                graph = self._graphs[(batch, bound)] = DecodeGraph(self, batch, bound)
            logits = graph.run(self.cache, requests, [int(p.tokens[0]) for p in portions], starts, slots)
            self.ops.launches += graph.kernels
            self.h2d_bytes_last = graph.nbytes
            self.graph_replays += 1
            wanted = [i for i, p in enumerate(portions) if len(p.want)]
            if not wanted:
                logits = None
            elif len(wanted) != batch:
                logits = logits[torch.tensor(wanted, device=self.device)]
            else:
                logits = logits.clone()          # the graph's own buffer is overwritten by the next replay
            num_tokens = batch
        else:
            tables = [self.cache.block_table(g, requests) for g in range(len(self.cache.groups))]
            ctx, rows, h2d = build_context(portions, starts, slots, tables, self.device)
            self.h2d_bytes_last = h2d
            logits = self.model.forward(ctx, rows)
            num_tokens = ctx.num_tokens
        for portion, start in zip(portions, starts):
            self.cache.set_computed(portion.request, start + len(portion.tokens))
        self.steps += 1
        self.tokens_run += num_tokens
        return logits


class DecodeGraph:
    """One CUDA graph of a decode step for a fixed number of requests.

    All index arrays live in one static device buffer that is refilled from a
    pinned host buffer before each replay; launch geometry is captured for a
    context bound (a power of two), and blocks whose key range is empty return
    at once, so one graph serves every context length up to its bound.
    """

    def __init__(self, runner: "ModelRunner", batch: int, max_ctx: int):
        from ..parts.base import StepContext
        self.batch = batch
        self.max_ctx = max_ctx
        model, cache = runner.model, runner.cache
        device = runner.device
        self.width = -(-max_ctx // cache.page_size)
        groups = len(cache.groups)
        sizes = [("token_ids", batch), ("positions", batch), ("seq_of_token", batch), ("q_start", batch + 1),
                 ("start_pos", batch), ("ctx_len", batch), ("slots", batch), ("rows", batch)]
        sizes += [(f"table{g}", batch * self.width) for g in range(groups)]
        self.offsets, cursor = {}, 0
        for name, count in sizes:
            self.offsets[name] = (cursor, count)
            cursor += count
        # A ring of pinned staging buffers: the host may fill the next one while earlier copies are
        # still queued; a buffer is reused only after the copy that read it has finished.
        self.ring = 4
        self.hosts = [torch.zeros(cursor, dtype=torch.int32).pin_memory() for _ in range(self.ring)]
        self.copied = [None] * self.ring
        self.turn = 0
        self.dev = torch.zeros(cursor, dtype=torch.int32, device=device)
        view = lambda t, name: t[self.offsets[name][0]:self.offsets[name][0] + self.offsets[name][1]]
        self.hs = [{name: view(host, name) for name, _ in sizes} for host in self.hosts]
        self.np_hs = [{name: tensor.numpy() for name, tensor in h.items()} for h in self.hs]   # same memory, cheap to fill
        d = {name: view(self.dev, name) for name, _ in sizes}
        for h in self.hs:
            # constants of a decode step
            h["seq_of_token"].copy_(torch.arange(batch, dtype=torch.int32))
            h["q_start"].copy_(torch.arange(batch + 1, dtype=torch.int32))
            h["rows"].copy_(torch.arange(batch, dtype=torch.int32))
            # warm-up contents: every request one token at position 0 on the scratch page
            h["ctx_len"].fill_(1)
            for g, group in enumerate(cache.groups):
                h[f"table{g}"].fill_(group.pool.capacity)
        self.dev.copy_(self.hosts[0])
        self.nbytes = cursor * 4
        self.ctx = StepContext(
            num_tokens=batch, num_seqs=batch, token_ids=d["token_ids"], positions=d["positions"],
            seq_of_token=d["seq_of_token"], q_start=d["q_start"], start_pos=d["start_pos"], ctx_len=d["ctx_len"],
            slots=d["slots"], block_tables=[d[f"table{g}"].view(batch, self.width) for g in range(groups)],
            max_q_len=1, max_ctx_len=max_ctx, typical_ctx_len=max_ctx // 2 + 1, host_q_lens=[1] * batch, host_start_pos=[0] * batch,
            host_slots=[0] * batch)
        self.rows = d["rows"]
        ops = runner.ops
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(2):
                model.forward(self.ctx, self.rows)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        before = ops.launches
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = model.forward(self.ctx, self.rows)
        self.kernels = ops.launches - before
        ops.launches = before

    def run(self, cache: CacheManager, requests, tokens, positions, slots) -> torch.Tensor:
        turn = self.turn
        self.turn = (turn + 1) % self.ring
        if self.copied[turn] is not None:
            self.copied[turn].synchronize()
        h = self.np_hs[turn]
        h["token_ids"][:] = tokens
        h["positions"][:] = positions
        h["start_pos"][:] = positions
        h["ctx_len"][:] = positions
        h["ctx_len"] += 1
        h["slots"][:] = slots
        for g in range(len(cache.groups)):
            cache.fill_block_table(g, requests, h[f"table{g}"].reshape(self.batch, self.width))
        self.dev.copy_(self.hosts[turn], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.copied[turn] = event
        self.graph.replay()
        return self.logits

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

import ctypes
from typing import Callable, Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import runtime as _rt
from ..cache.manager import CacheManager
from ..cache.pages import PoolExhausted
from ..models.decoder import DecoderModel
from .batch import Portion, PortionArrays, context_from_packed

# packs the step's index arrays: (fixed table width or 0, rows to pad to or 0, int32 buffer, layout) -> ints used
Packer = Callable[[int, int, np.ndarray, "_rt.StepLayout"], int]


class Staging:
    """A ring of pinned host buffers.  The host fills the next one while earlier copies are still queued;
    a buffer is used again only after the copy that read it has finished."""

    def __init__(self, ints: int, ring: int = 4):
        self.ring = ring
        self.hosts = [torch.zeros(ints, dtype=torch.int32).pin_memory() for _ in range(ring)]
        self.views = [host.numpy() for host in self.hosts]
        self.copied: List[Optional[torch.cuda.Event]] = [None] * ring
        self.turn = 0

    def take(self, ints: int = 0) -> int:
        """The next buffer's index, free to be written, at least ``ints`` long."""
        turn = self.turn
        self.turn = (turn + 1) % self.ring
        if self.copied[turn] is not None:
            self.copied[turn].synchronize()
            self.copied[turn] = None
        if self.hosts[turn].numel() < ints:
            self.hosts[turn] = torch.zeros(max(ints, 2 * self.hosts[turn].numel()), dtype=torch.int32).pin_memory()
            self.views[turn] = self.hosts[turn].numpy()
        return turn

    def queued(self, turn: int) -> None:
        """Call after the copy out of buffer ``turn`` was queued on the current stream."""
        event = torch.cuda.Event()
        event.record()
        self.copied[turn] = event


def graph_batch(batch: int) -> int:
    """The batch size whose decode graph serves ``batch`` single tokens: the next of 1, 2, 4, 8, 12, 16, 24,
    32, 48, 64, 96, 128, ... (powers of two and, from 8 on, the sizes halfway between).  An idle row costs a
    row of each product and one key, far less than capturing one more graph."""
    power = 1 << max(batch - 1, 0).bit_length()    # the next power of two at or above
    middle = power // 2 + power // 4
    return middle if 8 < batch <= middle else power


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_model_len: int, use_graphs: bool = True,
                 max_graph_batch: int = 256, max_graphs: int = 24):
        """``use_graphs``: steps made only of single tokens replay a CUDA graph captured per batch size and
        context bound.  Batch sizes are rounded up to a few sizes (:func:`graph_batch`) and the step is padded
        with idle rows, so that a batch that shrinks request by request does not capture a graph per size.
        At most ``max_graphs`` are kept (the one used longest ago goes first); all of them allocate from one
        memory pool, which is safe because replays never overlap: they run one after the other on the step's
        stream."""
        self.use_graphs = use_graphs and model.graph_safe      # a part that works from host values runs eagerly
        self.max_graph_batch = max_graph_batch
        self.max_graphs = max_graphs
        self._graphs: Dict[tuple, "DecodeGraph"] = {}          # in order of last use
        self._graph_pool = None
        self._capture_stream = None
        self.graphs_captured = 0
        self.graph_replays = 0
        self.model = model
        self.cache = cache
        self.max_model_len = max_model_len
        self.device = model.env.device
        self.ops = model.env.ops
        self.steps = 0
        self.tokens_run = 0
        self.h2d_bytes_last = 0
        self._lib = _rt.lib()
        self._staging: Optional[Staging] = None
        self._widest = -(-max_model_len // cache.page_size)

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
        cache, lib = self.cache, self._lib
        arrays = PortionArrays(cache, portions)
        fresh = [r for r in arrays.requests if not cache.is_live(r)] if cache.state_storage else []
        vocab = self.model.spec.vocab_size

        def pack(width: int, pad_rows: int, out: np.ndarray, layout) -> int:
            # admits unknown requests and grows pages, all or nothing, then writes the arrays
            return _rt.check(lib.tge_rt_step_pack(cache.native, arrays.count, arrays.handles, arrays.token_ptrs,
                                                  arrays.token_counts, arrays.want_ptrs, arrays.want_counts, vocab,
                                                  self.max_model_len, width, pad_rows, out.ctypes.data, out.size,
                                                  ctypes.byref(layout)))

        def packed() -> None:
            for request in fresh:                 # a request that starts gets a zeroed state slot
                cache.zero_state(cache.slot_of(request))

        max_ctx = lib.tge_rt_cache_max_context(cache.native, arrays.handles, arrays.token_counts, arrays.count)
        tokens = int(sum(arrays.token_counts))
        wanted = [i for i, w in enumerate(arrays.wants) if w.size]
        try:
            logits = self._run(pack, arrays.count, tokens, arrays.single_tokens, max_ctx, wanted, packed)
        except (PoolExhausted, ValueError):
            cache.forget_dead_handles()
            raise
        _rt.check(lib.tge_rt_cache_advance(cache.native, arrays.handles, arrays.token_counts, arrays.count))
        return logits

    def step_plan(self, plan) -> Optional[torch.Tensor]:
        """Runs a scheduler's plan: the same step, packed from the scheduler's own copies of the tokens.

        Pages were reserved when the plan was made, and the scheduler records progress in ``update``.
        """
        items = plan.items
        if not items:
            return None
        vocab = self.model.spec.vocab_size
        single = all(item.count == 1 for item in items)
        max_ctx = max(item.start + item.count for item in items)
        tokens = sum(item.count for item in items)
        wanted = [i for i, item in enumerate(items) if item.samples]
        return self._run(lambda width, pad_rows, out, layout: plan.pack(vocab, width, pad_rows, out, layout),
                         len(items), tokens, single, max_ctx, wanted, None)

    def can_step_ahead(self, batch: int) -> bool:
        return self.use_graphs and batch <= self.max_graph_batch

    def step_ahead(self, requests: Sequence[Hashable], token_ids: torch.Tensor) -> torch.Tensor:
        """One more token for each of ``requests`` (each already advanced past its previous step), the
        token ids taken from ``token_ids`` on the device: the step can be queued before the host has seen them.

        Pages are reserved all or nothing (PoolExhausted if they do not fit); progress is not recorded.
        Returns the logits of every row.
        """
        cache, lib = self.cache, self._lib
        count = len(requests)
        handles = (ctypes.c_int64 * count)(*[cache.handle_of(r) for r in requests])
        dummy = np.zeros(count, dtype=np.int32)
        want = np.zeros(count, dtype=np.int32)
        token_ptrs = (ctypes.c_void_p * count)(*[dummy.ctypes.data + 4 * i for i in range(count)])
        want_ptrs = (ctypes.c_void_p * count)(*[want.ctypes.data + 4 * i for i in range(count)])
        ones = (ctypes.c_int * count)(*([1] * count))
        vocab = self.model.spec.vocab_size

        def pack(width: int, pad_rows: int, out: np.ndarray, layout) -> int:
            return _rt.check(lib.tge_rt_step_pack(cache.native, count, handles, token_ptrs, ones, want_ptrs, ones, vocab,
                                                  self.max_model_len, width, pad_rows, out.ctypes.data, out.size,
                                                  ctypes.byref(layout)))

        max_ctx = lib.tge_rt_cache_max_context(cache.native, handles, ones, count)
        return self._run(pack, count, count, True, max_ctx, list(range(count)), None, device_tokens=token_ids)

    def _run(self, pack: Packer, batch: int, tokens: int, single: bool, max_ctx: int, wanted: List[int],
             packed: Optional[Callable[[], None]], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        groups = len(self.cache.groups)
        if self.use_graphs and single and batch <= self.max_graph_batch:
            bound = 1024
            while bound < max_ctx:
                bound *= 2
            bound = min(bound, self.max_model_len)
            padded = min(graph_batch(batch), self.max_graph_batch)
            graph = self._graphs.pop((padded, bound), None)
            if graph is None:
                while len(self._graphs) >= self.max_graphs:
                    del self._graphs[next(iter(self._graphs))]
                if self._graph_pool is None:
                    self._graph_pool = torch.cuda.graph_pool_handle()
                graph = DecodeGraph(self, padded, bound)
                self.graphs_captured += 1
            self._graphs[(padded, bound)] = graph
            logits = graph.run(pack, packed, device_tokens)
            self.ops.launches += graph.kernels
            self.h2d_bytes_last = graph.nbytes
            self.graph_replays += 1
            if not wanted:
                logits = None
            elif len(wanted) != batch:
                logits = logits[torch.tensor(wanted, device=self.device)]
            else:
                logits = logits[:batch].clone()  # the graph's own buffer is overwritten by the next replay
        else:
            need = 4 * tokens + 4 * batch + 1 + groups * batch * self._widest
            if self._staging is None:
                self._staging = Staging(max(need, 1 << 14))
            staging = self._staging
            turn = staging.take(need)
            layout = _rt.StepLayout()
            total = pack(0, 0, staging.views[turn], layout)
            if packed is not None:
                packed()
            dev = staging.hosts[turn][:total].to(self.device, non_blocking=True)
            staging.queued(turn)
            self.h2d_bytes_last = total * 4
            ctx, rows = context_from_packed(dev, staging.views[turn], layout, groups)
            logits = self.model.forward(ctx, rows)
        self.steps += 1
        self.tokens_run += tokens
        return logits


class DecodeGraph:
    """One CUDA graph of a decode step for a fixed number of rows: requests, and idle rows behind them.

    All index arrays live in one static device buffer that is refilled from a
    pinned host buffer before each replay; launch geometry is captured for a
    context bound (a power of two), and blocks whose key range is empty return
    at once, so one graph serves every context length up to its bound.
    """

    def __init__(self, runner: "ModelRunner", batch: int, max_ctx: int):
        self.batch = batch
        self.max_ctx = max_ctx
        model, cache = runner.model, runner.cache
        device = runner.device
        self.width = -(-max_ctx // cache.page_size)
        groups = len(cache.groups)
        # the packer's layout for `batch` single tokens, tables `width` wide, rows padded to `batch`
        L = self.layout = _rt.StepLayout()
        cursor = 0
        for name, count in (("token_ids", batch), ("positions", batch), ("seq_of_token", batch), ("q_start", batch + 1),
                            ("start_pos", batch), ("ctx_len", batch), ("slots", batch), ("logit_rows", batch)):
            setattr(L, name, cursor)
            cursor += count
        for g in range(groups):
            L.table[g], L.width[g] = cursor, self.width
            cursor += batch * self.width
        L.num_tokens = L.num_seqs = L.num_rows = batch
        L.max_q_len, L.max_ctx_len, L.total_ints = 1, max_ctx, cursor
        self.staging = Staging(cursor)
        self.dev = torch.zeros(cursor, dtype=torch.int32, device=device)
        # warm-up contents: every request one token at position 0 on the scratch page, its state in the scratch slot
        warm = self.staging.views[0]
        warm[L.slots:L.slots + batch] = cache.scratch_slot
        warm[L.seq_of_token:L.seq_of_token + batch] = np.arange(batch)
        warm[L.q_start:L.q_start + batch + 1] = np.arange(batch + 1)
        warm[L.logit_rows:L.logit_rows + batch] = np.arange(batch)
        warm[L.ctx_len:L.ctx_len + batch] = 1
        for g, group in enumerate(cache.groups):
            warm[L.table[g]:L.table[g] + batch * self.width] = group.pool.capacity
        self.dev.copy_(self.staging.hosts[0])
        self.nbytes = cursor * 4
        self.ctx, _ = context_from_packed(self.dev, warm, L, groups, max_ctx_len=max_ctx, typical_ctx_len=max_ctx // 2 + 1)
        # all rows' logits are computed; the rows a step wants are picked afterwards
        self.rows = torch.arange(batch, dtype=torch.int32, device=device)
        ops = runner.ops
        # Two eager steps first, on the step's own stream, whose cached blocks they reuse (on a stream of their
        # own every buffer was a new allocation from the driver: 6 ms became 40 to 150 now and then); then the
        # capture, on one side stream that all captures share.
        for _ in range(2):
            model.forward(self.ctx, self.rows)
        torch.cuda.synchronize(device)
        if runner._capture_stream is None:
            runner._capture_stream = torch.cuda.Stream(device=device)
        side = runner._capture_stream
        before = ops.launches
        self.graph = torch.cuda.CUDAGraph()
        try:
            self._capture(runner, side)
        except torch.OutOfMemoryError:
            # the graphs' pool found no room: give back what the allocator only caches, once, and try again
            torch.cuda.synchronize(device)
            torch.cuda.empty_cache()
            self.graph = torch.cuda.CUDAGraph()
            self._capture(runner, side)
        self.kernels = ops.launches - before
        ops.launches = before

    def _capture(self, runner: "ModelRunner", side: "torch.cuda.Stream") -> None:
        """Captures one step on a side stream into the graphs' shared pool.  (``torch.cuda.graph`` would first
        collect garbage and empty the allocator's cache: with requests in flight that took 30 to 500 ms per
        capture, most of it freeing and later re-allocating blocks that the steps in between use.)"""
        device = runner.device
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            self.graph.capture_begin(pool=runner._graph_pool)
            try:
                self.logits = runner.model.forward(self.ctx, self.rows)
            finally:
                self.graph.capture_end()
        torch.cuda.current_stream(device).wait_stream(side)

    def run(self, pack: Packer, packed: Optional[Callable[[], None]],
            device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        staging = self.staging
        turn = staging.take()
        layout = _rt.StepLayout()
        total = pack(self.width, self.batch, staging.views[turn], layout)
        if total != self.layout.total_ints or layout.table[0] != self.layout.table[0]:
            raise RuntimeError("decode graph: the packed step does not have the captured layout")
        if packed is not None:
            packed()
        self.dev.copy_(staging.hosts[turn], non_blocking=True)
        staging.queued(turn)
        if device_tokens is not None:      # the token ids are still on the device: they overwrite the packed placeholders
            first = self.layout.token_ids
            self.dev[first:first + device_tokens.numel()].copy_(device_tokens, non_blocking=True)
        self.graph.replay()
        return self.logits

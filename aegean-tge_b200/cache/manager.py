"""Cache manager: paged per-token cache in groups, and fixed-size state slots.

Layers whose mixers declare the same :class:`PagedCacheSpec` form a *group*.
A group has its own page pool, and one page id of the group addresses the same
page in every layer of the group, so a request has one block table per group,
not per layer.  Groups with a window give pages back as soon as no later
query can read them.  Beside the pages, every live request owns one *state
slot*: a row in each fixed-size state tensor that mixers with state declare
(this architecture's attention declares none; the slot still exists and is
what ``StepContext.slots`` carries).

The reference ships a contiguous ``[sequence][layer][context][kv_dim]`` cache
(src/models/qwen2.cpp:537-556) and a block table that is not wired in
(include/tge/models/block_table.hpp:3-9); its load-time planner shrinks the
context or refuses the load rather than run out (src/models/plan.cpp:72-124).
Here running out is a run-time event that the scheduler handles; this module
only answers "does it fit" and moves pages.

All bookkeeping is host-side and needs no GPU.  It is done in C++
(csrc/runtime.cpp: ``TgeRtCache``); this class maps request ids to the runtime's
64-bit handles, owns the storage tensors that ``allocate_storage`` creates, and
forwards everything else.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import runtime as _rt
from ..parts.base import LayerCache, PagedCacheSpec, StateSpec
from .pages import PageError, PagePool, PoolExhausted

NO_PAGE = -1


class _Tables:
    """Read-only view of one group's block tables: request -> list of physical page ids."""

    def __init__(self, manager: "CacheManager", group: int):
        self._manager, self._group = manager, group

    def __getitem__(self, request: Hashable) -> List[int]:
        m = self._manager
        if request not in m._handles:
            raise KeyError(request)
        handle = m._handles[request]
        length = _rt.check(m._lib.tge_rt_cache_table_length(m._cache, self._group, handle))
        out = (ctypes.c_int * max(length, 1))()
        _rt.check(m._lib.tge_rt_cache_table(m._cache, self._group, handle, out, length))
        return list(out[:length])

    def __contains__(self, request: Hashable) -> bool:
        return self._manager.is_live(request)

    def keys(self) -> Tuple[Hashable, ...]:
        return self._manager.live_requests()

    def values(self) -> Iterator[List[int]]:
        return (self[request] for request in self.keys())

    def items(self) -> Iterator[Tuple[Hashable, List[int]]]:
        return ((request, self[request]) for request in self.keys())

    def __len__(self) -> int:
        return len(self.keys())


@dataclass
class PageGroup:
    spec: PagedCacheSpec
    layers: List[int]
    page_size: int
    pool: PagePool
    tables: _Tables
    storage: Dict[str, torch.Tensor] = field(default_factory=dict)      # name -> [layers, pages, ...]

    def bytes_per_page(self, element_size: int) -> int:
        per_token = 0
        for _, shape in self.spec.entries:
            count = 1
            for d in shape:
                count *= d
            per_token += count
        return per_token * self.page_size * element_size * len(self.layers)

    def first_needed_page(self, computed_tokens: int) -> int:
        """Index of the first logical page a query at position >= computed_tokens can still read."""
        if self.spec.window is None:
            return 0
        first_key = max(computed_tokens - self.spec.window + 1, 0)
        return first_key // self.page_size


class CacheManager:
    def __init__(self, page_size: int, max_requests: int):
        if page_size <= 0 or max_requests <= 0:
            raise ValueError("cache manager: page_size and max_requests must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self._lib = _rt.lib()
        self._cache = self._lib.tge_rt_cache_create(int(page_size), int(max_requests))
        self.groups: List[PageGroup] = []
        self.layer_group: Dict[int, int] = {}                # layer id -> group index
        self.layer_row: Dict[int, int] = {}                  # layer id -> row in the group's storage
        self.state_specs: Dict[int, StateSpec] = {}          # layer id -> its state
        self.state_storage: Dict[int, Dict[str, torch.Tensor]] = {}
        # request id <-> the runtime's handle; a mapping lives while the request is live here or pinned
        # by the scheduler
        self._handles: Dict[Hashable, int] = {}
        self._names: Dict[int, Hashable] = {}
        self._pinned: set = set()
        self._next_handle = 1

    def __del__(self):
        if getattr(self, "_cache", None):
            self._lib.tge_rt_cache_destroy(self._cache)
            self._cache = None

    # -- request ids ------------------------------------------------------------
    def handle_of(self, request: Hashable, create: bool = False) -> int:
        handle = self._handles.get(request)
        if handle is None:
            if not create:
                raise PageError(f"cache manager: request {request!r} is not live")
            handle = self._next_handle
            self._next_handle += 1
            self._handles[request] = handle
            self._names[handle] = request
        return handle

    def name_of(self, handle: int) -> Hashable:
        return self._names[handle]

    def pin(self, request: Hashable) -> int:
        """Keeps the request's handle although it holds nothing here (the scheduler's waiting queue)."""
        handle = self.handle_of(request, create=True)
        self._pinned.add(request)
        return handle

    def unpin(self, request: Hashable) -> None:
        self._pinned.discard(request)
        self._drop_handle(request)

    def _drop_handle(self, request: Hashable) -> None:
        if request in self._pinned or request not in self._handles:
            return
        if self._lib.tge_rt_cache_is_live(self._cache, self._handles[request]):
            return
        self._names.pop(self._handles.pop(request), None)

    # -- construction ---------------------------------------------------------
    def add_layer(self, layer: int, cache: Optional[PagedCacheSpec], state: Optional[StateSpec]) -> None:
        """Declares what one layer keeps.  Layers with equal paged specs share a group."""
        if cache is not None:
            for index, group in enumerate(self.groups):
                if group.spec.group_key() == cache.group_key():
                    self.layer_group[layer] = index
                    self.layer_row[layer] = len(group.layers)
                    group.layers.append(layer)
                    break
            else:
                index = _rt.check(self._lib.tge_rt_cache_add_group(self._cache, -1 if cache.window is None else int(cache.window)))
                assert index == len(self.groups)
                self.layer_group[layer] = index
                self.layer_row[layer] = 0
                pool = PagePool(_borrowed=self._lib.tge_rt_cache_pool(self._cache, index))
                self.groups.append(PageGroup(cache, [layer], self.page_size, pool, _Tables(self, index)))
        if state is not None:
            self.state_specs[layer] = state

    def set_pool_sizes(self, pages_per_group: Sequence[int]) -> None:
        if len(pages_per_group) != len(self.groups):
            raise ValueError("cache manager: one page count per group")
        if self._lib.tge_rt_cache_live_count(self._cache):
            raise RuntimeError("cache manager: pools cannot be resized while requests are live")
        for index, (group, count) in enumerate(zip(self.groups, pages_per_group)):
            _rt.check(self._lib.tge_rt_cache_set_pool_size(self._cache, index, int(count)))
            group.pool = PagePool(_borrowed=self._lib.tge_rt_cache_pool(self._cache, index))

    def plan_pool_sizes(self, *, tokens: Optional[int] = None, budget_bytes: Optional[int] = None,
                        element_size: int = 2) -> List[int]:
        """Pages per group, either for ``tokens`` cached positions or from a byte budget.

        With a byte budget every group gets the same number of pages (a windowed
        group then simply never fills its share); with ``tokens`` each group
        gets ``ceil(tokens / page_size)``.
        """
        if not self.groups:
            return []
        if tokens is not None:
            pages = max(-(-tokens // self.page_size), 1)
            return [pages] * len(self.groups)
        if budget_bytes is None:
            raise ValueError("cache manager: give tokens or budget_bytes")
        per_page = sum(g.bytes_per_page(element_size) for g in self.groups)
        pages = budget_bytes // per_page
        if pages < 1:
            raise PoolExhausted(f"cache manager: {budget_bytes} bytes do not hold one page of every group "
                                f"({per_page} bytes)")
        return [int(pages)] * len(self.groups)

    def allocate_storage(self, dtype: torch.dtype, device: torch.device) -> None:
        """Creates the page and state tensors (zero-filled, so stale pages hold finite values).

        Every group gets one page more than its pool hands out (id ``capacity``): a scratch
        page that warm-up runs may write without touching a live request.  The state tensors likewise
        have one row more than there are slots (:attr:`scratch_slot`).
        """
        for group in self.groups:
            group.storage = {}
            for name, shape in group.spec.entries:
                full = (len(group.layers), group.pool.capacity + 1, *shape[:-1], self.page_size, shape[-1])
                group.storage[name] = torch.zeros(full, dtype=dtype, device=device)
        self.state_storage = {}
        for layer, spec in self.state_specs.items():
            self.state_storage[layer] = {
                name: torch.zeros((self.max_requests + 1, *shape), dtype=torch.float32, device=device)
                for name, shape in spec.entries}

    def layer_cache(self, layer: int, source: Optional[int] = None) -> LayerCache:
        """The views a layer's mixer works on; ``source`` names the layer whose pages it reads instead."""
        cache = LayerCache()
        holder = layer if source is None else source
        if holder in self.layer_group:
            group_index = self.layer_group[holder]
            group = self.groups[group_index]
            row = self.layer_row[holder]
            cache.group = group_index
            cache.paged = {name: tensor[row] for name, tensor in group.storage.items()}
            cache.owner = source is None
        if layer in self.state_storage:
            cache.state = self.state_storage[layer]
        return cache

    # -- requests -------------------------------------------------------------
    @property
    def native(self):
        """The runtime's cache object (for the scheduler and the step packer)."""
        return self._cache

    @property
    def free_slots(self) -> int:
        return self._lib.tge_rt_cache_free_slots(self._cache)

    def live_requests(self) -> Tuple[Hashable, ...]:
        count = self._lib.tge_rt_cache_live_count(self._cache)
        out = (ctypes.c_int64 * max(count, 1))()
        self._lib.tge_rt_cache_live_requests(self._cache, out, count)
        return tuple(self._names[h] for h in out[:count])

    def slot_of(self, request: Hashable) -> int:
        return _rt.check(self._lib.tge_rt_cache_slot_of(self._cache, self._live_handle(request)))

    def tokens_of(self, request: Hashable) -> int:
        return _rt.check(self._lib.tge_rt_cache_tokens_of(self._cache, self._live_handle(request)))

    def is_live(self, request: Hashable) -> bool:
        handle = self._handles.get(request)
        return handle is not None and bool(self._lib.tge_rt_cache_is_live(self._cache, handle))

    def _live_handle(self, request: Hashable) -> int:
        handle = self._handles.get(request)
        if handle is None:
            raise KeyError(request)
        return handle

    def computed(self, request: Hashable) -> int:
        """Tokens of the request whose cache entries have been written by finished steps."""
        return _rt.check(self._lib.tge_rt_cache_computed(self._cache, self._live_handle(request)))

    def set_computed(self, request: Hashable, tokens: int) -> None:
        """Records progress (never backwards) and gives back pages a window has passed."""
        _rt.check(self._lib.tge_rt_cache_set_computed(self._cache, self.handle_of(request), int(tokens)))

    def admit(self, request: Hashable) -> int:
        """Gives the request a state slot (zeroed) and empty block tables."""
        fresh = request not in self._handles
        try:
            slot = _rt.check(self._lib.tge_rt_cache_admit(self._cache, self.handle_of(request, create=True)))
        except Exception:
            if fresh:
                self._drop_handle(request)
            raise
        self.zero_state(slot)
        return slot

    def zero_state(self, slot: int) -> None:
        for tensors in self.state_storage.values():
            for tensor in tensors.values():
                tensor[slot].zero_()

    @property
    def scratch_slot(self) -> int:
        """A state row that belongs to no request: where warm-up runs and graph captures keep their state."""
        return self.max_requests

    def snapshot_state(self, slots: Sequence[int]) -> Optional[Tuple[torch.Tensor, List[torch.Tensor]]]:
        """Copies of the state rows of ``slots`` (None when no layer keeps state), for :meth:`restore_state`."""
        if not self.state_storage:
            return None
        tensors = [t for layer in self.state_storage.values() for t in layer.values()]
        index = torch.tensor(list(slots), dtype=torch.long, device=tensors[0].device)
        return index, [t.index_select(0, index) for t in tensors]

    def restore_state(self, snapshot: Optional[Tuple[torch.Tensor, List[torch.Tensor]]]) -> None:
        """Puts the rows of a snapshot back: a step that ran ahead and is dropped must leave no trace in state
        that is updated in place (pages need nothing: what it wrote lies beyond the recorded lengths)."""
        if snapshot is None:
            return
        index, rows = snapshot
        tensors = [t for layer in self.state_storage.values() for t in layer.values()]
        for tensor, saved in zip(tensors, rows):
            tensor.index_copy_(0, index, saved)

    def pages_missing(self, request: Hashable, total_tokens: int, computed_tokens: Optional[int] = None) -> List[int]:
        """Per group, pages that must be allocated so the request covers ``total_tokens`` positions."""
        out = (ctypes.c_int * 8)()
        handle = self._handles.get(request, 0)
        count = self._lib.tge_rt_cache_pages_missing(self._cache, handle, int(total_tokens), out)
        return list(out[:count])

    def can_grow(self, request: Hashable, total_tokens: int) -> bool:
        return bool(self._lib.tge_rt_cache_can_grow(self._cache, self._handles.get(request, 0), int(total_tokens)))

    def fits_empty_pool(self, total_tokens: int) -> bool:
        """Whether a request of this many tokens could ever fit, alone, in every pool.

        A windowed group holds at most the pages its window spans plus the
        pages a step's portion adds, which never exceeds the full count.
        """
        return bool(self._lib.tge_rt_cache_fits_empty_pool(self._cache, int(total_tokens)))

    def grow(self, request: Hashable, total_tokens: int) -> None:
        """Allocates pages so that positions [0, total_tokens) are covered.  All or nothing."""
        _rt.check(self._lib.tge_rt_cache_grow(self._cache, self.handle_of(request), int(total_tokens)))

    def release_behind_window(self, request: Hashable, computed_tokens: int) -> int:
        """Gives back pages that no query at position >= computed_tokens can read.  Returns how many."""
        return _rt.check(self._lib.tge_rt_cache_release_behind_window(self._cache, self.handle_of(request),
                                                                      int(computed_tokens)))

    def free(self, request: Hashable) -> None:
        """Gives back everything the request holds."""
        if request not in self._handles:
            raise PageError(f"cache manager: request {request!r} is not live (freed twice?)")
        _rt.check(self._lib.tge_rt_cache_free(self._cache, self._handles[request]))
        self._drop_handle(request)

    def forget_dead_handles(self) -> None:
        """Drops id mappings of requests the runtime freed on its own (the scheduler finishing a request)."""
        for request in [r for r in self._handles if r not in self._pinned]:
            self._drop_handle(request)

    def fill_block_table(self, group_index: int, requests: Sequence[Hashable], out: "np.ndarray") -> None:
        """Writes the requests' page ids into ``out`` (int32 [len(requests), width]), NO_PAGE beyond each row's end."""
        handles = (ctypes.c_int64 * len(requests))(*[self.handle_of(r) for r in requests])
        assert out.dtype == np.int32 and out.flags["C_CONTIGUOUS"]
        _rt.check(self._lib.tge_rt_cache_fill_block_table(self._cache, group_index, handles, len(requests),
                                                          out.ctypes.data, out.shape[1]))

    def block_table(self, group_index: int, requests: Sequence[Hashable], width: Optional[int] = None) -> List[List[int]]:
        """Rows of physical page ids, padded with NO_PAGE to a common width."""
        rows = [self.groups[group_index].tables[r] for r in requests]
        width = max([len(r) for r in rows] + [1]) if width is None else width
        return [row + [NO_PAGE] * (width - len(row)) for row in rows]

    def check(self) -> None:
        """No page lost, held twice, or free while referenced; slots consistent."""
        _rt.check(self._lib.tge_rt_cache_check(self._cache))

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

All bookkeeping is host-side and needs no GPU; the storage tensors are
created by ``allocate_storage``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import LayerCache, PagedCacheSpec, StateSpec
from .pages import PageError, PagePool, PoolExhausted

NO_PAGE = -1


@dataclass
class PageGroup:
    spec: PagedCacheSpec
    layers: List[int]
    page_size: int
    pool: PagePool
    tables: Dict[Hashable, List[int]] = field(default_factory=dict)    # request -> logical page -> physical id
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
        self.groups: List[PageGroup] = []
        self.layer_group: Dict[int, int] = {}                # layer id -> group index
        self.layer_row: Dict[int, int] = {}                  # layer id -> row in the group's storage
        self.state_specs: Dict[int, StateSpec] = {}          # layer id -> its state
        self.state_storage: Dict[int, Dict[str, torch.Tensor]] = {}
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}
        self._tokens: Dict[Hashable, int] = {}               # request -> tokens its pages cover
        self._computed: Dict[Hashable, int] = {}             # request -> tokens whose entries are written

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
                self.layer_group[layer] = len(self.groups)
                self.layer_row[layer] = 0
                self.groups.append(PageGroup(cache, [layer], self.page_size, PagePool(1)))
        if state is not None:
            self.state_specs[layer] = state

    def set_pool_sizes(self, pages_per_group: Sequence[int]) -> None:
        if len(pages_per_group) != len(self.groups):
            raise ValueError("cache manager: one page count per group")
        if self._slot_of:
            raise RuntimeError("cache manager: pools cannot be resized while requests are live")
        for group, count in zip(self.groups, pages_per_group):
            group.pool = PagePool(int(count))

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
        page that warm-up runs may write without touching a live request.
        """
        for group in self.groups:
            group.storage = {}
            for name, shape in group.spec.entries:
                full = (len(group.layers), group.pool.capacity + 1, *shape[:-1], self.page_size, shape[-1])
                group.storage[name] = torch.zeros(full, dtype=dtype, device=device)
        self.state_storage = {}
        for layer, spec in self.state_specs.items():
            self.state_storage[layer] = {
                name: torch.zeros((self.max_requests, *shape), dtype=torch.float32, device=device)
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
    def free_slots(self) -> int:
        return len(self._free_slots)

    def live_requests(self) -> Tuple[Hashable, ...]:
        return tuple(self._slot_of)

    def slot_of(self, request: Hashable) -> int:
        return self._slot_of[request]

    def tokens_of(self, request: Hashable) -> int:
        return self._tokens[request]

    def is_live(self, request: Hashable) -> bool:
        return request in self._slot_of

    def computed(self, request: Hashable) -> int:
        """Tokens of the request whose cache entries have been written by finished steps."""
        return self._computed[request]

    def set_computed(self, request: Hashable, tokens: int) -> None:
        """Records progress (never backwards) and gives back pages a window has passed."""
        if tokens > self._tokens[request]:
            raise PageError(f"cache manager: request {request!r} computed {tokens} tokens but holds pages for "
                            f"{self._tokens[request]}")
        if tokens > self._computed[request]:
            self._computed[request] = tokens
        self.release_behind_window(request, self._computed[request])

    def admit(self, request: Hashable) -> int:
        """Gives the request a state slot (zeroed) and empty block tables."""
        if request in self._slot_of:
            raise PageError(f"cache manager: request {request!r} is already live")
        if not self._free_slots:
            raise PoolExhausted("cache manager: no free state slot")
        slot = self._free_slots.pop()
        self._slot_of[request] = slot
        self._tokens[request] = 0
        self._computed[request] = 0
        for group in self.groups:
            group.tables[request] = []
        for tensors in self.state_storage.values():
            for tensor in tensors.values():
                tensor[slot].zero_()
        return slot

    def pages_missing(self, request: Hashable, total_tokens: int, computed_tokens: Optional[int] = None) -> List[int]:
        """Per group, pages that must be allocated so the request covers ``total_tokens`` positions."""
        missing = []
        need = -(-total_tokens // self.page_size)
        for group in self.groups:
            have = len(group.tables[request]) if request in group.tables else 0
            missing.append(max(need - have, 0))
        return missing

    def can_grow(self, request: Hashable, total_tokens: int) -> bool:
        return all(m <= g.pool.free_count for m, g in zip(self.pages_missing(request, total_tokens), self.groups))

    def fits_empty_pool(self, total_tokens: int) -> bool:
        """Whether a request of this many tokens could ever fit, alone, in every pool.

        A windowed group holds at most the pages its window spans plus the
        pages a step's portion adds, which never exceeds the full count.
        """
        need = -(-total_tokens // self.page_size)
        return all(need <= g.pool.capacity for g in self.groups)

    def grow(self, request: Hashable, total_tokens: int) -> None:
        """Allocates pages so that positions [0, total_tokens) are covered.  All or nothing."""
        if request not in self._slot_of:
            raise PageError(f"cache manager: request {request!r} is not live")
        missing = self.pages_missing(request, total_tokens)
        for m, group in zip(missing, self.groups):
            if m > group.pool.free_count:
                raise PoolExhausted(f"cache manager: request {request!r} needs {m} more pages, "
                                    f"{group.pool.free_count} are free")
        for m, group in zip(missing, self.groups):
            table = group.tables[request]
            for _ in range(m):
                table.append(group.pool.allocate())
        self._tokens[request] = max(self._tokens[request], total_tokens)

    def release_behind_window(self, request: Hashable, computed_tokens: int) -> int:
        """Gives back pages that no query at position >= computed_tokens can read.  Returns how many."""
        released = 0
        for group in self.groups:
            table = group.tables[request]
            for index in range(min(group.first_needed_page(computed_tokens), len(table))):
                if table[index] != NO_PAGE:
                    group.pool.release(table[index])
                    table[index] = NO_PAGE
                    released += 1
        return released

    def free(self, request: Hashable) -> None:
        """Gives back everything the request holds."""
        if request not in self._slot_of:
            raise PageError(f"cache manager: request {request!r} is not live (freed twice?)")
        for group in self.groups:
            for page in group.tables.pop(request):
                if page != NO_PAGE:
                    group.pool.release(page)
        self._free_slots.append(self._slot_of.pop(request))
        del self._tokens[request]
        del self._computed[request]

    def fill_block_table(self, group_index: int, requests: Sequence[Hashable], out: "np.ndarray") -> None:
        """Writes the requests' page ids into ``out`` (int32 [len(requests), width]), NO_PAGE beyond each row's end."""
        group = self.groups[group_index]
        out.fill(NO_PAGE)
        for row, request in enumerate(requests):
            table = group.tables[request]
            out[row, :len(table)] = table

    def block_table(self, group_index: int, requests: Sequence[Hashable], width: Optional[int] = None) -> List[List[int]]:
        """Rows of physical page ids, padded with NO_PAGE to a common width."""
        group = self.groups[group_index]
        rows = [group.tables[r] for r in requests]
        width = max([len(r) for r in rows] + [1]) if width is None else width
        return [row + [NO_PAGE] * (width - len(row)) for row in rows]

    def check(self) -> None:
        """No page lost, held twice, or free while referenced; slots consistent."""
        for group in self.groups:
            group.pool.check()
            held: Dict[int, int] = {}
            for request, table in group.tables.items():
                if request not in self._slot_of:
                    raise PageError(f"cache manager: a table exists for dead request {request!r}")
                for page in table:
                    if page != NO_PAGE:
                        held[page] = held.get(page, 0) + 1
            for page in range(group.pool.capacity):
                if group.pool.refcount(page) != held.get(page, 0):
                    raise PageError(f"cache manager: page {page} is held {held.get(page, 0)} times "
                                    f"but counts {group.pool.refcount(page)} references")
        slots = list(self._slot_of.values())
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("cache manager: a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise PageError("cache manager: a state slot is lost")

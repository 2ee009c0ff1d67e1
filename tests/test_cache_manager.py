"""Page pool, groups, windows and state slots (no GPU)."""
import random

import pytest
import torch

from aegean_tge_b200.cache import NO_PAGE, CacheManager, PageError, PagePool, PoolExhausted
from aegean_tge_b200.parts.base import PagedCacheSpec, StateSpec

FULL = PagedCacheSpec((("k", (2, 8)), ("v", (2, 8))), None)
WINDOW = PagedCacheSpec((("k", (2, 8)), ("v", (2, 8))), 40)


def _manager(pages=8, slots=4, specs=(FULL, FULL)):
    m = CacheManager(16, slots)
    for layer, spec in enumerate(specs):
        m.add_layer(layer, spec, None)
    m.set_pool_sizes([pages] * len(m.groups))
    return m


def test_pool_hands_out_the_page_freed_last():
    pool = PagePool(4)
    a, b = pool.allocate(), pool.allocate()
    assert (a, b) == (0, 1)
    assert pool.release(a) is True
    assert pool.allocate() == a                    # LIFO, as block_table.hpp's free list
    pool.check()


def test_pool_misuse_is_an_error():
    pool = PagePool(2)
    page = pool.allocate()
    pool.allocate()
    with pytest.raises(PoolExhausted):
        pool.allocate()
    pool.release(page)
    with pytest.raises(PageError):
        pool.release(page)                         # freed twice
    with pytest.raises(PageError):
        pool.share(page)                           # not live
    with pytest.raises(PageError):
        pool.release(7)
    pool.share(1)
    assert pool.release(1) is False and pool.refcount(1) == 1
    pool.check()


def test_layers_with_equal_needs_share_a_group():
    m = _manager(specs=(FULL, WINDOW, FULL, WINDOW, FULL))
    assert len(m.groups) == 2
    assert m.groups[0].layers == [0, 2, 4] and m.groups[1].layers == [1, 3]
    assert m.layer_group[3] == 1 and m.layer_row[4] == 2
    m.allocate_storage(torch.float32, torch.device("cpu"))
    assert m.groups[0].storage["k"].shape == (3, 8 + 1, 2, 16, 8)      # one scratch page beyond the pool
    view = m.layer_cache(2)
    assert view.group == 0 and view.paged["v"].shape == (9, 2, 16, 8) and view.owner
    shared = m.layer_cache(3, source=1)
    assert shared.group == 1 and not shared.owner
    assert shared.paged["k"].data_ptr() == m.layer_cache(1).paged["k"].data_ptr()


def test_grow_is_all_or_nothing_and_counts_pages():
    m = _manager(pages=5)
    m.admit("a")
    assert m.pages_missing("a", 33) == [3]
    m.grow("a", 33)
    assert m.groups[0].tables["a"] == [0, 1, 2] and m.pages_missing("a", 48) == [0]
    m.admit("b")
    assert not m.can_grow("b", 33)
    with pytest.raises(PoolExhausted):
        m.grow("b", 33)
    assert m.groups[0].tables["b"] == [] and m.groups[0].pool.free_count == 2
    m.grow("b", 32)
    m.check()
    m.free("a")
    assert m.groups[0].pool.free_count == 3
    m.grow("b", 70)                                # reuses a's pages, last freed first
    assert m.groups[0].tables["b"][2:] == [2, 1, 0]
    with pytest.raises(PageError):
        m.free("a")                                # freed twice
    m.check()


def test_block_table_rows_are_padded():
    m = _manager()
    m.admit("a"); m.admit("b")
    m.grow("a", 40); m.grow("b", 5)
    assert m.block_table(0, ["b", "a"]) == [[3, NO_PAGE, NO_PAGE], [0, 1, 2]]


def test_window_gives_pages_back_once_passed():
    m = _manager(pages=6, specs=(WINDOW,))
    m.admit("a")
    m.grow("a", 64)
    m.set_computed("a", 64)                        # next query at 64 reads keys >= 25: page 0 is dead
    assert m.groups[0].tables["a"] == [NO_PAGE, 1, 2, 3]
    assert m.groups[0].pool.free_count == 3
    m.grow("a", 96)
    m.set_computed("a", 96)                        # keys >= 57: pages 0..2 dead
    assert m.groups[0].tables["a"][:3] == [NO_PAGE] * 3
    m.check()
    m.free("a")
    assert m.groups[0].pool.free_count == 6
    m.check()


def test_window_edge_page_is_kept():
    m = _manager(pages=6, specs=(WINDOW,))
    m.admit("a")
    m.grow("a", 56)
    m.set_computed("a", 56)                        # first readable key 17: page 1 (16..31) must stay
    assert m.groups[0].tables["a"][:2] == [NO_PAGE, 1]
    m.set_computed("a", 55)                        # progress never goes backwards
    assert m.computed("a") == 56


def test_state_slots_are_zeroed_and_reused():
    m = CacheManager(16, 2)
    m.add_layer(0, None, StateSpec((("sum", (4,)),)))
    m.set_pool_sizes([])
    m.allocate_storage(torch.float32, torch.device("cpu"))
    a = m.admit("a")
    m.layer_cache(0).state["sum"][a] += 3.0
    m.admit("b")
    with pytest.raises(PoolExhausted):
        m.admit("c")
    with pytest.raises(PageError):
        m.admit("a")
    m.free("a")
    c = m.admit("c")
    assert c == a and float(m.layer_cache(0).state["sum"][c].abs().sum()) == 0.0
    m.check()


def test_pool_size_plans():
    m = _manager(specs=(FULL, WINDOW))
    assert m.plan_pool_sizes(tokens=100) == [7, 7]
    per_page = sum(g.bytes_per_page(2) for g in m.groups)
    assert per_page == 2 * (2 * 2 * 8 * 16 * 2)
    assert m.plan_pool_sizes(budget_bytes=per_page * 5 + 3, element_size=2) == [5, 5]
    with pytest.raises(PoolExhausted):
        m.plan_pool_sizes(budget_bytes=10, element_size=2)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Admit, grow, advance and free in random order: no page lost, held twice or freed twice."""
    rnd = random.Random(seed)
    m = _manager(pages=24, slots=5, specs=(FULL, WINDOW, FULL))
    live = {}
    for step in range(400):
        action = rnd.random()
        if action < 0.25 and m.free_slots and len(live) < 5:
            name = f"r{step}"
            m.admit(name)
            live[name] = 0
        elif action < 0.75 and live:
            name = rnd.choice(list(live))
            target = live[name] + rnd.randint(1, 40)
            if m.can_grow(name, target):
                m.grow(name, target)
                live[name] = target
                m.set_computed(name, target)
            else:
                with pytest.raises(PoolExhausted):
                    m.grow(name, target)
        elif live:
            name = rnd.choice(list(live))
            m.free(name)
            del live[name]
        m.check()
        for g in m.groups:
            held = sum(1 for t in g.tables.values() for p in t if p != NO_PAGE)
            assert held + g.pool.free_count == g.pool.capacity
    for name in list(live):
        m.free(name)
    m.check()
    assert all(g.pool.free_count == g.pool.capacity for g in m.groups) and m.free_slots == 5


def test_a_step_that_does_not_fit_takes_nothing():
    """The packer reserves a whole step or nothing: when the portions' pages do not fit in sum, requests that
    were live keep exactly what they had and requests that would have started are not admitted."""
    import ctypes

    import numpy as np

    from aegean_tge_b200 import runtime as rt
    from aegean_tge_b200.engine.batch import Portion, PortionArrays
    m = _manager(pages=6, slots=3, specs=(FULL, WINDOW))
    lib = rt.lib()

    def pack(portions):
        arrays = PortionArrays(m, portions)
        out = np.zeros(4096, dtype=np.int32)
        layout = rt.StepLayout()
        try:
            return rt.check(lib.tge_rt_step_pack(m.native, arrays.count, arrays.handles, arrays.token_ptrs,
                                                 arrays.token_counts, arrays.want_ptrs, arrays.want_counts, 100, 512, 0, 0,
                                                 out.ctypes.data, out.size, ctypes.byref(layout)))
        finally:
            m.forget_dead_handles()

    pack([Portion("a", [1] * 20, []), Portion("b", [2] * 10, [])])           # a: 2 pages, b: 1 page per group
    lib.tge_rt_cache_advance(m.native, (ctypes.c_int64 * 2)(m.handle_of("a"), m.handle_of("b")), (ctypes.c_int * 2)(20, 10), 2)
    before = [(g.pool.free_count, g.tables["a"], g.tables["b"]) for g in m.groups]
    # a grows by one page and b by one: fine alone, but c's three pages make it five where three are free
    with pytest.raises(PoolExhausted):
        pack([Portion("a", [1] * 20, []), Portion("b", [2] * 10, []), Portion("c", [3] * 40, [])])
    assert [(g.pool.free_count, g.tables["a"], g.tables["b"]) for g in m.groups] == before
    assert not m.is_live("c") and m.free_slots == 1
    m.check()
    # more new requests than slots: nothing is admitted either
    with pytest.raises(PoolExhausted):
        pack([Portion("c", [3], []), Portion("d", [4], [])])
    assert not m.is_live("c") and not m.is_live("d") and m.free_slots == 1
    assert [(g.pool.free_count, g.tables["a"], g.tables["b"]) for g in m.groups] == before
    pack([Portion("a", [1] * 20, []), Portion("b", [2] * 10, [])])           # the smaller step still runs
    m.check()


def test_a_padded_step_gets_idle_portions_on_the_scratch_page():
    """A step of single tokens packed for more rows than it has: the idle portions stand behind the real ones,
    one token at position 0, their tables name only the group's scratch page (id = capacity), their state is the
    scratch slot, and nothing is taken from the pools for them.  A step with a longer portion is not padded."""
    import ctypes

    import numpy as np

    from aegean_tge_b200 import runtime as rt
    from aegean_tge_b200.engine.batch import Portion, PortionArrays
    m = _manager(pages=6, slots=3, specs=(FULL, WINDOW))
    lib = rt.lib()

    def pack(portions, width, rows):
        arrays = PortionArrays(m, portions)
        out = np.full(4096, -7, dtype=np.int32)
        layout = rt.StepLayout()
        try:
            used = rt.check(lib.tge_rt_step_pack(m.native, arrays.count, arrays.handles, arrays.token_ptrs,
                                                 arrays.token_counts, arrays.want_ptrs, arrays.want_counts, 100, 512,
                                                 width, rows, out.ctypes.data, out.size, ctypes.byref(layout)))
        finally:
            m.forget_dead_handles()
        return out[:used], layout

    pack([Portion("a", [1] * 20, []), Portion("b", [2] * 3, [])], 0, 0)
    lib.tge_rt_cache_advance(m.native, (ctypes.c_int64 * 2)(m.handle_of("a"), m.handle_of("b")), (ctypes.c_int * 2)(20, 3), 2)
    free = [g.pool.free_count for g in m.groups]
    out, L = pack([Portion("a", [5], [0]), Portion("b", [6], [0])], 4, 5)
    assert (L.num_seqs, L.num_tokens, L.num_rows, L.max_q_len, L.max_ctx_len) == (5, 5, 2, 1, 21)
    assert L.total_ints == out.size and not (out == -7).any()             # every entry was written
    assert out[L.token_ids:L.token_ids + 5].tolist() == [5, 6, 0, 0, 0]
    assert out[L.positions:L.positions + 5].tolist() == [20, 3, 0, 0, 0]
    assert out[L.seq_of_token:L.seq_of_token + 5].tolist() == [0, 1, 2, 3, 4]
    assert out[L.q_start:L.q_start + 6].tolist() == [0, 1, 2, 3, 4, 5]
    assert out[L.start_pos:L.start_pos + 5].tolist() == [20, 3, 0, 0, 0]
    assert out[L.ctx_len:L.ctx_len + 5].tolist() == [21, 4, 1, 1, 1]
    assert out[L.slots:L.slots + 5].tolist() == [m.slot_of("a"), m.slot_of("b"), m.scratch_slot, m.scratch_slot, m.scratch_slot]
    for g, group in enumerate(m.groups):
        table = out[L.table[g]:L.table[g] + 5 * 4].reshape(5, 4)
        assert table[0, :2].tolist() == group.tables["a"][:2] and table[1, 0] == group.tables["b"][0]
        assert (table[2:] == np.array([group.pool.capacity, -1, -1, -1])).all()
    assert [g.pool.free_count for g in m.groups] == free                  # a's 21st token fits its second page
    m.check()
    with pytest.raises(ValueError, match="only a step of single tokens can be padded"):
        pack([Portion("a", [5, 6], [0]), Portion("b", [6], [0])], 4, 5)

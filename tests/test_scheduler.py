"""The scheduler's decisions, with a stand-in for the model (no GPU)."""
import pytest

from aegean_tge_b200.cache import CacheManager
from aegean_tge_b200.engine.scheduler import FINISHED, Request, Scheduler
from aegean_tge_b200.parts.base import PagedCacheSpec
from aegean_tge_b200.sampling import SamplingParams

SPEC = PagedCacheSpec((("k", (1, 8)), ("v", (1, 8))), None)


def _setup(pages, **kw):
    cache = CacheManager(16, kw.pop("slots", 4))
    cache.add_layer(0, SPEC, None)
    cache.set_pool_sizes([pages])
    kw.setdefault("max_batch_tokens", 64)
    kw.setdefault("max_requests", 4)
    kw.setdefault("max_model_len", 256)
    return cache, Scheduler(cache, **kw)


def _run(scheduler, cache, token_of=lambda request: 1000 + len(request.output), limit=1000):
    """Drives the scheduler as the engine does; the 'model' answers with a function of the request."""
    plans = []
    while scheduler.has_work():
        plan = scheduler.schedule()
        for item in plan.items:                                  # what the step function would check
            assert cache.computed(item.request.id) == item.start
            assert cache.tokens_of(item.request.id) >= item.start + item.count
        sampled = [token_of(item.request) for item in plan.items if item.samples]
        scheduler.update(plan, sampled)
        cache.check()
        plans.append(plan)
        assert len(plans) < limit
    return plans


def test_prompts_are_cut_under_the_token_budget():
    cache, s = _setup(64, max_batch_tokens=32)
    s.add(Request("a", list(range(70)), 3))
    plans = _run(s, cache)
    counts = [[(i.request.id, i.start, i.count, i.samples) for i in p.items] for p in plans]
    assert counts[:3] == [[("a", 0, 32, False)], [("a", 32, 32, False)], [("a", 64, 6, True)]]
    assert counts[3:] == [[("a", 70, 1, True)], [("a", 71, 1, True)]]
    assert s.finished["a"].output == [1000, 1001, 1002] and s.finished["a"].finish_reason == "length"
    assert cache.groups[0].pool.free_count == 64 and cache.free_slots == 4


def test_decodes_run_beside_prompt_portions():
    cache, s = _setup(64, max_batch_tokens=16, chunk=12)
    s.add(Request("a", list(range(5)), 4))
    s.add(Request("b", list(range(30)), 2))
    plans = _run(s, cache)
    first = [(i.request.id, i.count) for i in plans[0].items]
    assert first == [("a", 5), ("b", 11)]                       # budget 16: a whole, b's first 11
    second = [(i.request.id, i.count, i.samples) for i in plans[1].items]
    assert second == [("a", 1, True), ("b", 12, False)]          # a decodes, b's portion capped by chunk
    assert all(p.num_tokens <= 16 for p in plans)


def test_admission_is_in_arrival_order_and_bounded():
    cache, s = _setup(64, max_requests=2, max_batch_tokens=64)
    for name in "abc":
        s.add(Request(name, [1, 2, 3], 2))
    plan = s.schedule()
    assert [i.request.id for i in plan.items] == ["a", "b"]     # c waits for a slot
    s.update(plan, [7, 7])
    plan = s.schedule()
    s.update(plan, [7, 7])                                       # a and b finish
    plan = s.schedule()
    assert [i.request.id for i in plan.items] == ["c"]


def test_end_token_and_context_limit_finish_a_request():
    cache, s = _setup(64, end_token_ids=[9], max_model_len=8)
    s.add(Request("a", [1, 2, 3], 50))
    s.add(Request("b", [1, 2, 3, 4, 5], 50))
    _run(s, cache, token_of=lambda r: 9 if (r.id == "a" and len(r.output) == 2) else 5)
    assert s.finished["a"].output == [5, 5, 9] and s.finished["a"].finish_reason == "end_token"
    assert s.finished["b"].finish_reason == "context" and s.finished["b"].num_tokens == 8


def test_requests_that_can_never_fit_are_refused():
    cache, s = _setup(4)
    with pytest.raises(ValueError):
        s.add(Request("big", list(range(70)), 1))               # 5 pages > 4
    s.add(Request("ok", list(range(60)), 5))                    # 64 tokens cached at most: 4 pages
    with pytest.raises(ValueError):
        s.add(Request("ok", [1], 1))                            # id in use
    with pytest.raises(ValueError):
        s.add(Request("none", [], 1))
    with pytest.raises(ValueError):
        s.add(Request("bad", [1], 1, SamplingParams(top_p=1.5)))
    with pytest.raises(ValueError):
        s.add(Request("long", list(range(256)), 1))             # no room in the context


def test_when_pages_run_out_the_newest_request_is_preempted_and_recomputed():
    cache, s = _setup(6, max_batch_tokens=64)                    # 96 tokens of cache
    s.add(Request("a", list(range(40)), 30))                     # grows to 69 tokens: 5 pages
    s.add(Request("b", list(range(100, 130)), 30))               # grows to 59 tokens: 4 pages
    events = []
    plans = _run(s, cache)
    for p in plans:
        events += p.preempted
    assert "b" in events and "a" not in events                   # the most recently admitted one goes
    assert s.counters["preemptions"] >= 1
    a, b = s.finished["a"], s.finished["b"]
    assert a.output == [1000 + i for i in range(30)] and b.output == [1000 + i for i in range(30)]
    assert b.preemptions >= 1 and a.preemptions == 0
    # after preemption b was recomputed from its prompt plus what it had generated
    restart = next(i for p in plans for i in p.items if i.request.id == "b" and i.start == 0 and p is not plans[0])
    assert restart.count > 30
    assert cache.groups[0].pool.free_count == 6


def test_no_admission_in_a_step_that_preempted():
    cache, s = _setup(4, max_batch_tokens=64)
    s.add(Request("a", list(range(31)), 20))
    s.add(Request("b", list(range(31)), 20))
    s.add(Request("c", [1, 2], 2))
    for _ in range(200):
        if not s.has_work():
            break
        plan = s.schedule()
        if plan.preempted:
            admitted_now = [i.request.id for i in plan.items if i.start == 0 and i.request.preemptions == 0
                            and i.request.computed == 0 and i.request.id == "c"]
            assert not admitted_now or not [i for i in plan.items if i.request.id != "c"]
        s.update(plan, [5 for i in plan.items if i.samples])
        cache.check()
    assert not s.has_work() and set(s.finished) == {"a", "b", "c"}


def test_a_lone_request_that_fits_always_progresses():
    cache, s = _setup(3, max_batch_tokens=8, chunk=5)
    s.add(Request("a", list(range(40)), 9))                      # 48 tokens at most: exactly 3 pages
    plans = _run(s, cache)
    assert s.finished["a"].state == FINISHED and len(s.finished["a"].output) == 9
    assert all(not p.preempted for p in plans)


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_the_same_outputs_whatever_the_pool(seed):
    """Requests of random sizes arrive at random times into pools from roomy to barely sufficient, with random
    budgets and portion caps.  Every request finishes with the tokens a function of (request, position)
    dictates, nothing is lost or held twice on the way, and the packed step matches the plan."""
    import random

    import numpy as np

    from aegean_tge_b200 import runtime as rt
    rnd = random.Random(seed)
    specs = [(f"r{i}", rnd.randint(1, 70), rnd.randint(1, 25)) for i in range(rnd.randint(3, 12))]
    largest = max(-(-(p + n - 1) // 16) for _, p, n in specs)
    expected = {name: [(7 * len(name) + 13 * p + 31 * k) % 97 for k in range(n)] for name, p, n in specs}
    for pages in (largest, largest + 2, 64):
        cache, s = _setup(pages, slots=rnd.randint(1, 4), max_batch_tokens=rnd.choice([3, 8, 16, 64]),
                          max_requests=rnd.randint(1, 4), chunk=rnd.choice([None, 2, 5, 16]), max_model_len=128)
        arrivals = sorted((rnd.randint(0, 30), spec) for spec in specs)
        out = np.zeros(4096, dtype=np.int32)
        layout = rt.StepLayout()
        step = 0
        while arrivals or s.has_work():
            while arrivals and arrivals[0][0] <= step:
                _, (name, p, n) = arrivals.pop(0)
                s.add(Request(name, [(3 * i + len(name)) % 97 for i in range(p)], n))
            step += 1
            if not s.has_work():
                continue
            plan = s.schedule()
            assert plan.num_tokens <= s.max_batch_tokens and plan.items
            plan.pack(97, 0, 0, out, layout)
            assert layout.num_tokens == plan.num_tokens and layout.num_seqs == len(plan.items)
            assert layout.num_rows == sum(i.samples for i in plan.items)
            cursor = layout.token_ids
            for index, item in enumerate(plan.items):
                tokens = item.request.token_slice(item.start, item.count)
                assert out[cursor:cursor + item.count].tolist() == tokens
                assert out[layout.start_pos + index] == item.start == cache.computed(item.request.id)
                assert out[layout.slots + index] == cache.slot_of(item.request.id)
                table = cache.groups[0].tables[item.request.id]
                width = layout.width[0]
                row = out[layout.table[0] + index * width:layout.table[0] + (index + 1) * width].tolist()
                assert row[:len(table)] == table and all(x == -1 for x in row[len(table):])
                cursor += item.count
            sampled = [expected[i.request.id][len(i.request.output)] for i in plan.items if i.samples]
            s.update(plan, sampled)
            cache.check()
            assert step < 5000
        assert {name: s.finished[name].output for name in expected} == expected
        assert cache.free_slots == cache.max_requests and cache.groups[0].pool.free_count == pages
        assert not cache._handles, "id mappings of finished requests are dropped"

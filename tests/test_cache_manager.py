"""The cache manager's accounting (no GPU): no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots."""
import random

import numpy as np
import pytest

from beglin_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from beglin_b200.parts.cache_need import FixedStateNeed, PagedKVNeed


def test_pool_reuses_last_freed_first_and_refuses_double_free():
    p = PagePool(4)
    a = p.alloc(3)
    assert a == [0, 1, 2] and p.num_free == 1
    p.free([1])
    assert p.alloc(1) == [1]
    with pytest.raises(OutOfPages):
        p.alloc(2)
    assert p.num_free == 1                        # a refused allocation changes nothing
    p.free([0])
    with pytest.raises(CacheError):
        p.free([0])
    with pytest.raises(CacheError):
        p.free([7])
    p.check()


def manager(window=None, pages=8, page=4, reqs=3, extra=()):
    needs = [PagedKVNeed(2, 16), PagedKVNeed(2, 16), PagedKVNeed(2, 16, window)] + list(extra)
    return CacheManager(needs, page_size=page, num_pages=pages, max_requests=reqs)


def test_groups_by_need():
    m = manager(window=8, extra=[None, FixedStateNeed((4,)), FixedStateNeed((4,))])
    assert [g.stages for g in m.kv_groups] == [[0, 1], [2]]
    assert [g.stages for g in m.state_groups] == [[4, 5]]
    assert m.stage_group[1] == ("kv", 0, 1) and m.stage_group[5] == ("state", 0, 1) and 3 not in m.stage_group


def test_reserve_is_atomic_and_tables_grow():
    m = manager(pages=4, page=4)
    m.add_request("a")
    m.add_request("b")
    m.reserve([("a", 5), ("b", 4)])
    m.commit([("a", 5), ("b", 4)])
    assert m.block_table(0, ["a", "b"]).tolist()[0][:3] == [0, 1, -1]
    assert m.free_pages() == 1
    with pytest.raises(OutOfPages):
        m.reserve([("a", 9), ("b", 8)])          # needs 2, one free
    assert m.free_pages() == 1 and m.pages_held("a") == 2
    m.check()
    m.release("a")
    assert m.free_pages() == 3
    with pytest.raises(CacheError):
        m.release("a")
    m.reserve([("b", 12)])
    # page 1 then 0 come back first: what "a" held is used again
    assert m.block_table(0, ["b"]).tolist()[0][:3] == [2, 1, 0]
    m.check()


def test_window_gives_pages_back_as_it_passes_them():
    m = CacheManager([PagedKVNeed(1, 16, 6)], page_size=4, num_pages=4, max_requests=2, max_context=64)
    m.add_request("a")
    held = []
    for n in range(1, 40):                        # one token at a time, far beyond 4 pages of 4
        m.reserve([("a", n)])
        m.commit([("a", n)])
        held.append(m.pages_held("a"))
        t = m.kv_groups[0].tables["a"]
        first_query = n - 1
        lo = max(0, first_query - 6 + 1)
        for i, p in enumerate(t):
            assert (p >= 0) == (i >= lo // 4), (n, t)
        m.check()
    assert max(held) <= 3


def test_context_limit_and_unknown_requests():
    m = CacheManager([PagedKVNeed(1, 16)], page_size=4, num_pages=8, max_requests=1, max_context=10)
    with pytest.raises(CacheError):
        m.reserve([("x", 1)])
    m.add_request("x")
    with pytest.raises(CacheError, match="context limit"):
        m.reserve([("x", 11)])
    with pytest.raises(CacheError, match="slots"):
        m.add_request("y")
    m.reserve([("x", 10)])
    m.commit([("x", 10)])
    with pytest.raises(CacheError, match="shrink"):
        m.reserve([("x", 3)])


def test_slots_are_recycled():
    m = manager(reqs=2)
    s0, s1 = m.add_request("a"), m.add_request("b")
    assert {s0, s1} == {0, 1}
    m.release("a")
    assert m.add_request("c") == s0
    assert m.slot_ids(["c", "b"]).tolist() == [s0, s1]
    m.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(window=10, pages=12, page=4, reqs=4)
    live = {}
    nxt = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{nxt}"; nxt += 1
            m.add_request(rid); live[rid] = 0
        elif op < 0.4 and live:
            rid = rng.choice(list(live))
            m.release(rid); del live[rid]
        elif live:
            group = rng.sample(list(live), rng.randint(1, len(live)))
            plan = [(r, live[r] + rng.randint(1, 9)) for r in group]
            before = (m.free_pages(), {r: m.pages_held(r) for r in live})
            try:
                m.reserve(plan)
            except (OutOfPages, CacheError) as e:
                assert isinstance(e, OutOfPages) or "context limit" in str(e)
                assert before == (m.free_pages(), {r: m.pages_held(r) for r in live})
            else:
                m.commit(plan)
                for r, n in plan:
                    live[r] = n
        m.check()
        assert set(m.live()) == set(live)
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.free_pages() == 12


def test_a_request_that_starts_again_under_its_name_is_another_request():
    """Whoever remembers what the device holds for a request (a replayed graph) compares identities, not
    names: the same name after a release is a new request, with other pages in another order."""
    m = manager(pages=8, page=4, reqs=2)
    m.add_request("r"); m.add_request("s")
    m.reserve([("r", 5), ("s", 3)]); m.commit([("r", 5), ("s", 3)])
    first = m.identity(["r", "s"])
    assert m.identity(["r", "s"]) == first
    table = m.block_table(0, ["r"]).tolist()
    m.release("r")
    m.release("s")
    m.add_request("r")
    m.reserve([("r", 5)]); m.commit([("r", 5)])
    assert m.length("r") == 5 and m.identity(["r"]) != first[:1]        # same name, same length, another request
    assert m.block_table(0, ["r"]).tolist() != table                     # and its pages lie elsewhere
    m.check()


def test_trim_gives_back_what_a_step_that_did_not_happen_had_reserved():
    m = manager(window=6, pages=8, page=4, reqs=2)
    m.add_request("r")
    m.reserve([("r", 6)]); m.commit([("r", 6)])
    free = [g.pool.num_free for g in m.kv_groups]
    m.reserve([("r", 19)])                       # reserved for a step ...
    assert [g.pool.num_free for g in m.kv_groups] != free
    m.trim(["r", "not live"])                    # ... that failed
    assert [g.pool.num_free for g in m.kv_groups] == free and m.length("r") == 6
    m.check()
    m.reserve([("r", 7)]); m.commit([("r", 7)])  # and the request goes on
    m.check()


def test_spare_page_and_slot_are_never_handed_out():
    m = manager(pages=3, page=4, reqs=2, extra=[FixedStateNeed((2,))])
    for i in range(2):
        m.add_request(i)
    m.reserve([(0, 8), (1, 4)])
    held = {p for g in m.kv_groups for t in g.tables.values() for p in t}
    assert m.dump_page == 3 and m.dump_page not in held and max(held) < 3
    assert m.dump_slot == 2 and m.dump_slot not in m.slots.values()

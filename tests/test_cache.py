"""The cache manager without a GPU: no page lost, held twice or freed twice, under random orders of requests."""
import random

import pytest

from llmx_b200.cache import BlockTable, CacheExhausted, CacheManager, KVSpec, PagePool, RELEASED, StateSlots, StateSpec


def test_pool_allocates_each_page_once_and_refuses_double_free():
    pool = PagePool(4)
    got = [pool.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and pool.free_pages == 0
    with pytest.raises(CacheExhausted):
        pool.alloc()
    pool.release(got[1])
    with pytest.raises(RuntimeError, match="released twice"):
        pool.release(got[1])
    assert pool.alloc() == got[1]            # the page just given back is used again
    pool.retain(got[0])
    pool.release(got[0])
    assert pool.refs(got[0]) == 1
    with pytest.raises(RuntimeError):
        pool.retain(17 % 4 if pool.refs(1) == 0 else 99) if False else pool.release(99)
    pool.check()


def test_block_table_prepare_commit_abort():
    pool = PagePool(5)
    t = BlockTable(pool, page_size=4)
    t.prepare(6)
    assert len(t.pages) == 2 and t.pending == 6 and t.length == 0
    with pytest.raises(RuntimeError, match="already in progress"):
        t.prepare(1)
    t.commit()
    assert t.length == 6 and pool.used_pages == 2
    t.prepare(1)                              # fits the second page
    assert len(t.pages) == 2
    t.abort()
    assert t.length == 6 and len(t.pages) == 2
    t.prepare(3)                              # needs a third page
    assert len(t.pages) == 3
    t.abort()
    assert len(t.pages) == 2 and pool.used_pages == 2
    assert t.slot_of(5) == t.pages[1] * 4 + 1
    t.free()
    assert pool.used_pages == 0
    pool.check()


def test_exhaustion_gives_back_what_the_failed_prepare_took():
    pool = PagePool(3)
    a, b = BlockTable(pool, 4), BlockTable(pool, 4)
    a.prepare(8)
    a.commit()
    with pytest.raises(CacheExhausted):
        b.prepare(9)                          # would need 3 pages, one is free
    assert pool.used_pages == 2 and b.pages == [] and b.pending == 0
    b.prepare(4)
    b.commit()
    assert pool.free_pages == 0
    pool.check()


def test_window_gives_back_the_pages_it_has_passed():
    pool = PagePool(8)
    t = BlockTable(pool, page_size=4, window=6)
    for n in (5, 4, 4, 4, 4):
        t.prepare(n)
        t.commit()
    # 21 tokens: the next query (position 21) needs keys from 16 on, so pages 0..3 are gone.
    assert t.length == 21 and t.pages[:4] == [RELEASED] * 4 and t.held_pages == 2
    assert pool.used_pages == 2
    with pytest.raises(RuntimeError, match="given back"):
        t.slot_of(3)
    t.prepare(20)                             # a long portion: pages for it are taken, none of the live ones is lost
    t.commit()
    assert t.held_pages == pool.used_pages <= 3
    t.free()
    assert pool.used_pages == 0
    pool.check()


def test_state_slots():
    s = StateSlots(2)
    a, b = s.take(), s.take()
    assert {a, b} == {0, 1}
    with pytest.raises(CacheExhausted):
        s.take()
    s.give_back(a)
    with pytest.raises(RuntimeError, match="twice"):
        s.give_back(a)
    assert s.take() == a
    s.check()


def test_groups_by_need_and_all_or_nothing_prepare():
    specs = [KVSpec(2, 16), KVSpec(2, 16, window=8), KVSpec(2, 16), StateSpec((4, 3)), None, KVSpec(2, 16, window=8)]
    m = CacheManager(specs, page_size=4, kv_tokens=32, max_requests=3)
    assert len(m.groups) == 2 and m.groups[0].members == [0, 2] and m.groups[1].members == [1, 5]
    assert m.group_of_entry[5] == (1, 1) and m.state_entries == [3] and m.has_state
    a = m.new_request("a")
    assert a.state_slot == 0
    a.prepare(20)
    a.commit()
    assert m.used_pages() == [5, 2]           # the windowed group keeps the keys from position 13 on: pages 3 and 4
    b = m.new_request("b")
    with pytest.raises(CacheExhausted):
        b.prepare(16)                         # the full group has 3 pages left, the windowed one enough
    assert m.used_pages() == [5, 2] and b.pending == 0          # what the windowed group took went back
    m.check()
    with pytest.raises(RuntimeError, match="already live"):
        m.new_request("a")
    m.free_request("a")
    m.free_request("b")
    assert m.used_pages() == [0, 0] and m.state_slots.free_slots == 6      # two a request: its state and a spare
    m.check()
    assert m.pages_needed(100, step_tokens=4) == [25, 5]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_lose_no_page(seed):
    """Requests arrive, grow by portions and single tokens, fail for lack of room, end in any order."""
    rng = random.Random(seed)
    specs = [KVSpec(1, 8), KVSpec(1, 8, window=rng.choice([5, 16, 40])), StateSpec((2,))]
    m = CacheManager(specs, page_size=rng.choice([1, 4, 16]), kv_tokens=rng.choice([64, 96, 160]), max_requests=5)
    live, next_id, reused = {}, 0, set()
    ever_freed = [set(), set()]
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            live[next_id] = m.new_request(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            n = rng.choice([1, 1, 1, 2, 3, 7, 20, 50])
            before = m.used_pages()
            try:
                rc.prepare(n)
            except CacheExhausted:
                assert m.used_pages() == before and rc.pending == 0
            else:
                for g, t in enumerate(rc.tables):
                    reused |= {(g, p) for p in t.pages if p in ever_freed[g]}
                if rng.random() < 0.15:
                    rc.abort()
                    assert rc.length == rc.tables[0].length
                else:
                    rc.commit()
        elif live:
            rid = rng.choice(list(live))
            for g, t in enumerate(live[rid].tables):
                ever_freed[g] |= {p for p in t.pages if p != RELEASED}
            m.free_request(rid)
            del live[rid]
        m.check()
        for rc in live.values():
            assert rc.tables[0].held_pages == -(-rc.length // m.page_size)
    for rid in list(live):
        m.free_request(rid)
    m.check()
    assert m.used_pages() == [0, 0] and m.state_slots.free_slots == 10
    assert reused, "the run never used a page again; it did not test reuse"


def test_state_is_part_of_the_transaction_and_requests_roll_back():
    """A step reads a request's state slot and writes its spare; commit swaps them, abort does not, so a failed
    step leaves the state where it was.  A request without state can be rolled back to a shorter history."""
    from llmx_b200.cache.manager import CacheManager, KVSpec, StateSpec
    m = CacheManager([KVSpec(1, 8), StateSpec((4,))], page_size=4, kv_tokens=64, max_requests=2)
    a = m.new_request("a")
    first, spare = a.state_slot, a.state_slot_out
    assert first != spare and min(first, spare) >= 0 and m.state_slots.free_slots == 2
    a.prepare(5)
    a.abort()
    assert (a.state_slot, a.state_slot_out) == (first, spare) and a.length == 0
    a.prepare(5)
    a.commit()
    assert (a.state_slot, a.state_slot_out) == (spare, first) and a.length == 5
    with pytest.raises(RuntimeError, match="fixed-size state"):
        a.truncate(2)
    a.truncate(5)                                   # to where it is: nothing to do
    m.free_request("a")
    assert m.state_slots.free_slots == 4
    m.check()

    k = CacheManager([KVSpec(1, 8), KVSpec(1, 8, window=6)], page_size=4, kv_tokens=64, max_requests=2, window_kv_tokens=32)
    assert k.total_pages() == [16, 8]               # the windowed group's pool is its own size
    b = k.new_request("b")
    b.prepare(10)
    b.commit()
    used = k.used_pages()
    b.prepare(9)
    b.commit()
    assert b.length == 19
    with pytest.raises(RuntimeError, match="window has given back"):
        b.truncate(3)
    b.truncate(17)
    assert b.length == 17 and [t.length for t in b.tables] == [17, 17]
    k.check()
    with pytest.raises(ValueError):
        b.truncate(18)
    b.prepare(2)
    b.commit()
    assert b.length == 19
    k.free_request("b")
    assert k.used_pages() == [0, 0] and used != [0, 0]
    k.check()

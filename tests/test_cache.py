"""The cache manager and the state slots (host logic, no GPU): no page lost,
held twice or freed twice, under random orders of requests; windows give
pages back; a failed reservation takes nothing."""
from __future__ import annotations

import random

import pytest

from inferflux_b200.cache import KVCacheManager, OutOfPages, OutOfSlots, PagePool, StateSlotManager
from inferflux_b200.parts.base import KVNeed


def test_pool_alloc_free_reuse():
    p = PagePool(4)
    a = p.alloc(3)
    assert len(set(a)) == 3 and p.num_free == 1
    with pytest.raises(OutOfPages):
        p.alloc(2)
    assert p.num_free == 1                       # a refused request takes nothing
    p.free(a[:2])
    with pytest.raises(ValueError, match="freed twice"):
        p.free(a[:1])
    with pytest.raises(ValueError, match="not of this pool"):
        p.free([9])
    b = p.alloc(2)
    assert set(b) == set(a[:2]) and p.reuses == 2  # the pages just given back are used again
    p.check()


def test_block_tables_grow_by_pages():
    kv = KVCacheManager([KVNeed.keys_and_values(2, 16)], [8], 16)
    kv.add_request("a")
    assert kv.pages_needed("a", 1) == [1] and kv.pages_needed(None, 33) == [3]
    kv.reserve("a", 17)
    assert len(kv.block_table("a", 0)) == 2 and kv.length("a") == 0
    kv.advance("a", 17)
    assert kv.length("a") == 17 and kv.pages_needed("a", 15) == [0] and kv.pages_needed("a", 16) == [1]
    assert kv.slot_of("a", 0, 16) == kv.block_table("a", 0)[1] * 16
    with pytest.raises(RuntimeError, match="beyond the reserved"):
        kv.advance("a", 100)
    with pytest.raises(KeyError):
        kv.add_request("a")
    kv.free_request("a")
    assert kv.num_free(0) == 8
    kv.check()


def test_failed_reservation_takes_nothing():
    kv = KVCacheManager([KVNeed.keys_and_values(2, 16), KVNeed.keys_and_values(2, 16, window=8)], [10, 2], 4)
    kv.add_request("a")
    with pytest.raises(OutOfPages) as e:
        kv.reserve("a", 12)                      # group 1 has 2 pages, 3 are needed
    assert e.value.group == 1
    assert kv.num_free(0) == 10 and kv.num_free(1) == 2 and kv.block_table("a", 0) == []
    kv.check()


def test_window_gives_pages_back():
    w, ps = 10, 4
    kv = KVCacheManager([KVNeed.keys_and_values(1, 16), KVNeed.keys_and_values(1, 16, window=w)], [64, 64], ps)
    kv.add_request("a")
    length = 0
    for n in (7, 1, 1, 9, 2, 30, 1, 1, 1):
        kv.reserve("a", n)
        kv.advance("a", n)
        length += n
        full, win = kv.block_table("a", 0), kv.block_table("a", 1)
        assert all(p >= 0 for p in full) and len(full) == len(win) == (length + ps - 1) // ps
        first_key = max(0, length - w + 1)       # the oldest key the next token can still see
        for b, page in enumerate(win):
            assert (page < 0) == ((b + 1) * ps <= first_key), (length, b, win)
        kv.check()
    held = sum(1 for p in kv.block_table("a", 1) if p >= 0)
    assert held <= (w + ps - 1) // ps + 1
    kv.free_request("a")
    assert kv.num_free(0) == 64 and kv.num_free(1) == 64


def test_random_request_orders_lose_nothing():
    rng = random.Random(0)
    needs = [KVNeed.keys_and_values(2, 16), KVNeed.keys_and_values(1, 32, window=24)]
    for trial in range(30):
        ps = rng.choice([4, 16, 64])
        pages = [rng.randint(6, 40), rng.randint(6, 40)]
        kv = KVCacheManager(needs, pages, ps)
        slots = StateSlotManager(5)
        live, counter = {}, 0
        for _ in range(300):
            op = rng.random()
            if op < 0.25 and slots.num_free:
                rid = f"r{counter}"
                counter += 1
                kv.add_request(rid)
                slots.acquire(rid)
                live[rid] = 0
            elif op < 0.85 and live:
                rid = rng.choice(sorted(live))
                n = rng.choice([1, 1, 1, 2, 5, 17, 40])
                if kv.can_reserve(rid, n):
                    kv.reserve(rid, n)
                    kv.advance(rid, n)
                    live[rid] += n
                    assert kv.length(rid) == live[rid]
                else:
                    before = [kv.num_free(g) for g in range(2)]
                    with pytest.raises(OutOfPages):
                        kv.reserve(rid, n)
                    assert before == [kv.num_free(g) for g in range(2)]
            elif live:
                rid = rng.choice(sorted(live))
                kv.free_request(rid)
                slots.release(rid)
                del live[rid]
            kv.check()
            slots.check()
        for rid in list(live):
            kv.free_request(rid)
            slots.release(rid)
        kv.check()
        assert [kv.num_free(g) for g in range(2)] == pages and slots.num_free == 5


def test_state_slots():
    s = StateSlotManager(2)
    a, b = s.acquire("a"), s.acquire("b")
    assert a != b and s.num_free == 0
    with pytest.raises(OutOfSlots):
        s.acquire("c")
    with pytest.raises(KeyError):
        s.acquire("a")
    s.release("a")
    assert s.acquire("c") == a                  # the seat is used again
    s.check()


def test_table_stamp_changes_with_the_tables():
    """The stamp tells a holder of a copy of the block tables whether it is still right."""
    kv = KVCacheManager([KVNeed.keys_and_values(2, 16), KVNeed.keys_and_values(2, 16, window=20)], [8, 8], 16)
    kv.add_request("a")
    s0 = kv.table_stamp("a")
    kv.reserve("a", 10)
    s1 = kv.table_stamp("a")
    assert s1 != s0                                  # a page was taken
    kv.advance("a", 10)
    kv.reserve("a", 3)
    kv.advance("a", 3)
    assert kv.table_stamp("a") == s1                 # tokens within the page: the tables stand
    kv.reserve("a", 30)
    s2 = kv.table_stamp("a")
    kv.advance("a", 30)                              # 43 tokens: the window has passed block 0
    assert kv.block_table("a", 1)[0] == -1 and kv.table_stamp("a") not in (s1, s2)
    kv.free_request("a")
    kv.add_request("a")
    kv.reserve("a", 10)
    assert kv.table_stamp("a") not in (s0, s1, s2)   # the same name, another sequence
    kv.check()

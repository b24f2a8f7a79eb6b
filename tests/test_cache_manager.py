"""The cache manager on the host: no page lost, held twice or freed twice."""
import random

import pytest

from crucible_b200.cache import (CacheError, CacheManager, GroupPolicy, PagePool, PoolExhausted,
                                 RELEASED, StateSlotPool)


def test_pool_hands_out_each_page_once_and_takes_it_back_once():
    pool = PagePool(4, 16)
    pages = [pool.alloc() for _ in range(4)]
    assert pages == [0, 1, 2, 3] and pool.free_pages == 0
    with pytest.raises(PoolExhausted, match="exhausted"):
        pool.alloc()
    pool.release(2)
    with pytest.raises(CacheError, match="double free"):
        pool.release(2)
    with pytest.raises(CacheError, match="out of range"):
        pool.release(9)
    assert pool.alloc() == 2                       # a freed page is used again


def test_state_slots():
    slots = StateSlotPool(2)
    a, b = slots.acquire(), slots.acquire()
    assert {a, b} == {0, 1}
    with pytest.raises(PoolExhausted):
        slots.acquire()
    slots.release(a)
    with pytest.raises(CacheError):
        slots.release(a)
    assert slots.acquire() == a


def test_growth_is_lazy_and_all_or_nothing_across_groups():
    m = CacheManager([GroupPolicy(16), GroupPolicy(8)], [4, 5], n_state_slots=3)
    m.add_request("a")
    m.extend("a", 7)
    assert m.held_pages("a", 0) == 1 and m.held_pages("a", 1) == 1
    m.extend("a", 10)                                  # 17 tokens: 2 pages of 16, 3 of 8
    assert m.held_pages("a", 0) == 2 and m.held_pages("a", 1) == 3
    m.add_request("b")
    m.extend("b", 16)                                  # 1 page and 2 pages: group 1 is now full
    with pytest.raises(PoolExhausted):
        m.extend("a", 16)                              # group 0 has room, group 1 has not
    assert m.length("a") == 17
    assert m.held_pages("a", 0) == 2 and m.free_pages(0) == 1      # rolled back
    m.check_invariants()
    m.remove_request("b")
    m.extend("a", 15)
    assert m.length("a") == 32
    m.remove_request("a")
    assert m.free_pages(0) == 4 and m.free_pages(1) == 5 and m.slots.free_slots == 3
    with pytest.raises(CacheError):
        m.remove_request("a")


def test_reservations_keep_room_for_admitted_requests():
    m = CacheManager([GroupPolicy(16)], [8], n_state_slots=4)
    assert m.can_reserve(100)                 # 7 pages
    m.add_request("a", lifetime_tokens=100)
    assert m.reserved_pages(0) == 7
    assert not m.can_reserve(32)              # 2 pages, 1 unreserved
    assert m.can_reserve(16)
    with pytest.raises(PoolExhausted):
        m.add_request("b", lifetime_tokens=32)
    assert not m.has("b") and m.slots.free_slots == 3      # refusal changed nothing
    m.add_request("c", lifetime_tokens=16)
    assert not m.can_reserve(1)
    m.remove_request("a")
    assert m.reserved_pages(0) == 1 and m.can_reserve(100)
    assert not m.fits_at_all(16 * 8 + 1) and m.fits_at_all(16 * 8)


def test_window_group_gives_back_pages_the_window_has_passed():
    m = CacheManager([GroupPolicy(16), GroupPolicy(16, window=20)], [32, 4], n_state_slots=2)
    m.add_request("a")
    m.extend("a", 30)                # positions 0..29; next token 30 reads keys from 11
    assert m.held_pages("a", 1) == 2
    m.extend("a", 10)                # at 30: block 0 (0..15) still holds key 11..15 -> kept
    assert m.block_table("a", 1)[0] != RELEASED and m.held_pages("a", 1) == 3
    m.extend("a", 1)                 # at 40: first needed key 21 -> block 0 released
    assert m.block_table("a", 1)[0] == RELEASED and m.held_pages("a", 1) == 2
    for _ in range(200):             # a long decode never needs more than 3 pages of the window group
        m.extend("a", 1)
        assert m.held_pages("a", 1) <= 3
        m.check_invariants()
    assert m.held_pages("a", 0) == -(-m.length("a") // 16)      # the full group keeps everything
    assert m.pages_for(1, 10_000, max_step_tokens=1) <= 3
    m.remove_request("a")
    assert m.free_pages(1) == 4 and m.free_pages(0) == 32


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    m = CacheManager([GroupPolicy(16), GroupPolicy(4, window=9)], [24, 30], n_state_slots=5)
    live = {}
    for step in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            rid = f"r{step}"
            m.add_request(rid)
            live[rid] = 0
        elif action < 0.85 and live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 33])
            before = (m.length(rid), m.held_pages(rid, 0))
            try:
                m.extend(rid, n)
                live[rid] += n
            except PoolExhausted:
                assert m.length(rid) == before[0] and m.held_pages(rid, 0) == before[1]
        elif live:
            rid = rng.choice(sorted(live))
            m.remove_request(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.length(rid) == n
            table = m.block_table(rid, 0)
            assert len(table) == -(-n // 16) and RELEASED not in table
    for rid in list(live):
        m.remove_request(rid)
    assert m.free_pages(0) == 24 and m.free_pages(1) == 30 and m.slots.free_slots == 5


def _manager_with_rows():
    return CacheManager([GroupPolicy(16), GroupPolicy(4, window=9)], [12, 10], n_state_slots=3,
                        table_strides=[8, 32], null_pages=[12, 10])


def test_device_rows_follow_the_tables():
    """The row that goes to the device: the table's pages, the null page where a page was
    given back early, zeros beyond the table and after the request has gone."""
    m = _manager_with_rows()
    m.add_request("a")
    rng = random.Random(5)
    for _ in range(40):
        m.extend("a", rng.choice([1, 2, 3, 5]))
        for g, null in ((0, 12), (1, 10)):
            table = m.block_table("a", g)
            row = m.table_row("a", g)
            assert list(row[:len(table)]) == [null if p == RELEASED else p for p in table]
            assert not row[len(table):].any()
    assert RELEASED in m.block_table("a", 1)
    m.shrink("a", 3)
    table = m.block_table("a", 1)
    assert len(table) == -(-m.length("a") // 4)
    assert not m.table_row("a", 1)[len(table):].any()
    m.check_invariants()
    m.check_tables()
    slot = m.state_slot("a")
    m.remove_request("a")
    m.add_request("b")
    assert m.state_slot("b") == slot and not m.table_row("b", 0).any()


def test_a_table_that_outgrows_its_row_is_refused():
    m = CacheManager([GroupPolicy(16)], [12], n_state_slots=2, table_strides=[8], null_pages=[12])
    m.add_request("a")                             # rows of 8 entries: 128 tokens
    m.extend("a", 100)
    with pytest.raises(CacheError, match="table entries"):
        m.extend("a", 29)
    assert m.length("a") == 100
    m.extend("a", 28)
    m.check_invariants()


def test_a_step_grows_every_request_or_none():
    m = CacheManager([GroupPolicy(16)], [6], n_state_slots=4, table_strides=[6], null_pages=[6])
    for r in "abc":
        m.add_request(r)
    assert m.extend_step(["a", "b", "c"], [20, 5, 16]) == [0, 0, 0]        # 2 + 1 + 1 pages
    assert m.extend_step(["c", "a"], [1, 1]) == [16, 20]                   # c takes a 5th page
    free = m.free_pages(0)
    with pytest.raises(PoolExhausted, match="request 'b'"):
        m.extend_step(["a", "b", "c"], [12, 30, 1])                        # a fits, b does not
    assert [m.length(r) for r in "abc"] == [21, 5, 17] and m.free_pages(0) == free
    with pytest.raises(CacheError, match="context"):
        m.extend_step(["a", "b"], [1, 60], max_tokens=64)
    assert [m.length(r) for r in "abc"] == [21, 5, 17] and m.free_pages(0) == free
    with pytest.raises(CacheError, match="not live"):
        m.extend_step(["a", "zz"], [1, 1])
    m.check_invariants()
    m.check_tables()


def test_a_page_handed_out_twice_is_seen_before_it_is_shared():
    """The allocator at fault (a held page put back on the free stack): the growth that
    would put the page into a second table is refused and leaves everything as it was."""
    m = _manager_with_rows()
    m.add_request("a")
    m.extend("a", 20)
    m.add_request("b")
    held = m.block_table("a", 0)[1]
    m.pools[0].release(held)
    free = [m.free_pages(0), m.free_pages(1)]
    with pytest.raises(CacheError, match="another live request"):
        m.extend("b", 40)                          # takes `held` first, then would take more
    assert m.length("b") == 0 and m.block_table("b", 0) == [] and m.block_table("b", 1) == []
    assert [m.free_pages(0), m.free_pages(1)] == free
    assert m.pools[0].alloc() == held              # the stack reads as the fault left it
    m.check_invariants()
    m.check_tables()
    # a table entry changed behind the manager's back is found by the whole check
    m.extend("b", 5)
    m._poke("b", 0, 0, m.block_table("a", 0)[0])
    with pytest.raises(CacheError, match="'b' and request 'a'|'a' and request 'b'"):
        m.check_tables()


@pytest.mark.parametrize("seed", range(4))
def test_random_steps_with_rows_and_rollbacks(seed):
    rng = random.Random(100 + seed)
    m = CacheManager([GroupPolicy(8), GroupPolicy(4, window=6)], [14, 12], n_state_slots=4,
                     table_strides=[40, 80], null_pages=[14, 12])
    lengths = {}
    for step in range(400):
        if len(lengths) < 4 and rng.random() < 0.3:
            rid = f"r{step}"
            m.add_request(rid)
            lengths[rid] = 0
        if lengths and rng.random() < 0.1:
            rid = rng.choice(sorted(lengths))
            m.remove_request(rid)
            del lengths[rid]
        if not lengths:
            continue
        who = rng.sample(sorted(lengths), rng.randint(1, len(lengths)))
        counts = [rng.choice([1, 1, 2, 9, 17]) for _ in who]
        try:
            first = m.extend_step(who, counts, max_tokens=300)
            assert first == [lengths[r] for r in who]
            for r, n in zip(who, counts):
                lengths[r] += n
            if rng.random() < 0.2:                 # what a failed packer would cause
                for r, n in zip(reversed(who), reversed(counts)):
                    m.shrink(r, n)
                    lengths[r] -= n
        except PoolExhausted:
            pass
        except CacheError as e:
            assert "context" in str(e)
        m.check_invariants()
        m.check_tables()
        for r, n in lengths.items():
            assert m.length(r) == n
            for g, (pt, null) in enumerate(((8, 14), (4, 12))):
                table = m.block_table(r, g)
                assert len(table) == -(-n // pt)
                row = m.table_row(r, g)
                assert list(row[:len(table)]) == [null if p == RELEASED else p for p in table]
    for r in list(lengths):
        m.remove_request(r)
    assert m.free_pages(0) == 14 and m.free_pages(1) == 12 and m.slots.free_slots == 4

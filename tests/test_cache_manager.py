"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""

import random

import pytest

from fastgen_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from fastgen_b200.parts.base import CacheSpec, StateSpec


def manager(n_pages=16, page=8, window=None, max_requests=4, max_length=256, two_groups=False):
    full = CacheSpec(2, 16, None)
    specs = [full, full]
    kv_from = [None, None]
    if window or two_groups:
        specs += [CacheSpec(2, 16, window or 20), CacheSpec(2, 16, window or 20), full]
        kv_from += [None, None, 0]
    return CacheManager(specs, [None] * len(specs), kv_from, page, n_pages, max_requests, max_length)


def test_pool_order_and_double_free():
    pool = PagePool(5)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.n_free == 2
    pool.give([1])
    assert pool.take(1) == [1]
    with pytest.raises(CacheError):
        pool.give([4])  # never handed out
    pool.give(a)
    with pytest.raises(CacheError):
        pool.give([0])  # freed twice
    with pytest.raises(OutOfPages):
        pool.take(6)
    assert pool.n_free == 5


def test_groups_and_sharing():
    m = manager(two_groups=True)
    assert len(m.groups) == 2
    assert m.groups[0].entries == [0, 1] and m.groups[1].entries == [2, 3]
    assert m.entry_group[4] == 0 and m.entry_index[4] == 0  # entry 4 reads entry 0's cache
    assert m.memory(4).writes is False and m.memory(0).writes is True


def test_reserve_advance_release():
    m = manager()
    r = m.admit("a")
    assert m.pages_needed(r, 9) == [2]
    m.reserve(r, 9)
    m.advance(r, 9)
    assert m.free_pages() == [14] and r.length == 9
    m.reserve(r, 16)  # still inside the second page
    assert m.free_pages() == [14]
    m.reserve(r, 17)
    assert m.free_pages() == [13]
    m.check()
    m.release("a")
    assert m.free_pages() == [16] and m.free_slots() == 4
    with pytest.raises(CacheError):
        m.release("a")
    m.check()


def test_reserve_is_atomic_across_groups():
    full, win = CacheSpec(2, 16, None), CacheSpec(1, 16, 20)
    m = CacheManager([full, win], [None, None], [None, None], 8, [8, 2], 4, 256)
    r = m.admit("a")
    with pytest.raises(OutOfPages):
        m.reserve(r, 30)  # the windowed group only has 2 pages; 4 are needed for one portion
    assert m.free_pages() == [8, 2]
    m.check()


def test_window_gives_pages_back():
    m = manager(window=20, n_pages=32)
    r = m.admit("a")
    held = []
    for length in range(1, 120):
        m.reserve(r, length)
        m.advance(r, length)
        held.append(len(r.pages[1]))
        m.check()
        # every key a query at position >= length may see still has its page
        for j in range(max(0, length - 20 + 1), length):
            assert j // 8 in r.pages[1]
    assert max(held) <= 4  # window 20 over pages of 8: at most 4 pages
    assert len(r.pages[0]) == 15  # the full group keeps everything
    m.release("a")
    assert m.free_pages() == [32, 32]


def test_limits():
    m = manager(n_pages=4, max_requests=2, max_length=64)
    a = m.admit("a")
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.admit("c")
    with pytest.raises(CacheError):
        m.admit("a")
    with pytest.raises(OutOfPages):
        m.reserve(a, 33)  # 5 pages of 8
    with pytest.raises(OutOfPages):
        m.reserve(a, 65)  # beyond max_length
    assert m.free_pages() == [4]
    assert m.can_ever_hold(32) and not m.can_ever_hold(33)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_invariants(seed):
    rng = random.Random(seed)
    m = manager(n_pages=24, window=20 if seed % 2 else None, two_groups=bool(seed % 2), max_requests=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            live[next_id] = m.admit(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            r = live[rid]
            new_len = r.length + rng.choice([1, 1, 1, 2, 5, 16, 21])
            try:
                m.reserve(r, new_len)
                m.advance(r, new_len)
            except OutOfPages:
                before = m.free_pages()
                m.release(rid)  # "preempt"
                del live[rid]
                assert all(a >= b for a, b in zip(m.free_pages(), before))
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(f == g.pool.n_pages for f, g in zip(m.free_pages(), m.groups))
    assert m.free_slots() == 4


def test_groups_with_pages_of_their_own_and_one_pool():
    """A spec may ask for its own page size and for a single pool: such runs form a group with its
    own page ids, block-table width and byte count; one ``n_pages`` gives every group the same tokens."""
    kv = CacheSpec(2, 16, None)
    latent = CacheSpec(1, 12, None, n_pools=1, page_size=4)
    windowed = CacheSpec(2, 16, 10, page_size=2)
    m = CacheManager([kv, latent, kv, windowed], [None] * 4, [None] * 4, page_size=8, n_pages=6, max_requests=3,
                     max_length=48)
    assert [g.page_size for g in m.groups] == [8, 4, 2]
    assert [g.pool.n_pages for g in m.groups] == [6, 12, 24]
    assert [g.table_width for g in m.groups] == [6, 12, 24]
    assert [g.bytes_per_token(2) for g in m.groups] == [2 * 2 * 2 * 16 * 2, 1 * 1 * 1 * 12 * 2, 2 * 1 * 2 * 16 * 2]
    assert m.memory(1).page_size == 4 and m.memory(0).page_size == 8
    r = m.admit("a")
    assert m.pages_needed(r, 9) == [2, 3, 5]
    m.reserve(r, 9)
    m.advance(r, 9)
    m.check()
    m.reserve(r, 30)
    m.advance(r, 30)
    # the windowed group gave back what the window (10 keys) has passed, in pages of 2
    assert m.free_pages() == [6 - 4, 12 - 8, 24 - 5]
    m.check()
    assert m.can_ever_hold(48) and not m.can_ever_hold(49)
    m.release("a")
    assert m.free_pages() == [6, 12, 24]
    with pytest.raises(ValueError):
        CacheSpec(1, 8, None, n_pools=3)

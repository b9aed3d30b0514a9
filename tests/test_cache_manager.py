"""The cache manager on the host: arithmetic of reserve/commit/close (the cases of
the reference's engine/kv/kv_test.go), all-or-nothing reservations, groups with
pages of their own, windows that give pages back, state slots, and random orders
of requests under which no page is lost, held twice or freed twice."""
import random

import pytest
import torch

from kllm_b200.cache import CacheError, CacheManager, IdPool, OutOfPages
from kllm_b200.parts.spec import PagedKVNeed, StateNeed

FULL = PagedKVNeed(n_kv_heads=2, head_dim=16)


def manager(needs=None, page_size=4, num_pages=8, max_requests=4, allocate=False):
    return CacheManager(needs or [FULL, FULL], page_size, num_pages, max_requests, allocate=allocate)


def test_reserve_commit_close_arithmetic():
    m = manager()
    r = m.open()
    m.reserve(r, 5)                       # 5 tokens, pages of 4 -> 2 pages
    assert r.tables[0] == [0, 1] and r.length == 0
    m.commit(r, 5)
    assert r.length == 5
    m.reserve(r, 3)                       # 8 tokens still fit 2 pages
    assert len(r.tables[0]) == 2
    m.commit(r, 3)
    m.reserve(r, 1)                       # the 9th token needs a third
    assert r.tables[0] == [0, 1, 2]
    m.commit(r, 1)
    assert m.free_pages() == [5]
    m.close(r)
    assert m.free_pages() == [8] and r.closed
    m.audit()


def test_out_of_pages_then_reuse_last_freed_first():
    m = manager(num_pages=4)
    a, b = m.open(), m.open()
    m.reserve(a, 8)
    m.commit(a, 8)
    m.reserve(b, 8)
    m.commit(b, 8)
    c = m.open()
    with pytest.raises(OutOfPages):
        m.reserve(c, 1)
    assert c.tables[0] == []
    m.close(a)                            # pages 0, 1 come back
    m.reserve(c, 5)
    assert sorted(c.tables[0]) == [0, 1] and c.tables[0][0] == 1    # LIFO: the last freed goes out first
    m.audit()


def test_tables_are_disjoint():
    m = manager(num_pages=8)
    rs = [m.open() for _ in range(3)]
    for r, n in zip(rs, (7, 9, 4)):
        m.reserve(r, n)
    pages = [p for r in rs for p in r.tables[0]]
    assert len(pages) == len(set(pages)) == 2 + 3 + 1
    m.audit()


def test_reservation_is_all_or_nothing_over_groups():
    window = PagedKVNeed(2, 16, window=6)
    m = manager(needs=[FULL, window, FULL], num_pages=3)
    assert len(m.groups) == 2 and m.groups[0].slots == [0, 2] and m.groups[1].slots == [1]
    a = m.open()
    m.reserve(a, 8)                        # 2 pages in each group
    b = m.open()
    with pytest.raises(OutOfPages):
        m.reserve(b, 5)                    # needs 2, one free in each group
    assert b.tables == [[], []] and m.free_pages() == [1, 1]
    assert not m.can_reserve(b, 5) and m.can_reserve(b, 4)
    assert not m.can_reserve_all([(a, 12), (b, 1)]) and m.can_reserve_all([(a, 12)])
    assert m.room_for(b) == 4 and m.room_for(a) == 12 and m.room_for(b, [1, 0]) == 0
    m.audit()


def test_pool_size_from_a_byte_budget_over_two_groups():
    """pages = budget / bytes of one page in every pool: two layers that keep all keys
    (2 kv heads of 16), one window layer with another shape (1 kv head of 32), bfloat16,
    pages of 4 tokens; a fixed count ran out of memory in the reference
    (docs/JOURNAL.md:364-367)."""
    other = PagedKVNeed(1, 32, window=6)
    needs = [FULL, other, FULL, StateNeed((3,))]
    per = (2 * 2 * 2 * 4 * 16 + 1 * 2 * 1 * 4 * 32) * 2          # layers * (k, v) * heads * slots * dim * bytes
    assert CacheManager(needs, 4, 1, 2, dtype=torch.bfloat16, allocate=False).bytes_per_page() == per
    assert CacheManager.pages_within(needs, 4, torch.bfloat16, 10 * per + per - 1) == 10
    assert CacheManager.pages_within(needs, 4, torch.float32, 10 * per) == 5
    with pytest.raises(ValueError, match="holds no page"):
        CacheManager.pages_within(needs, 4, torch.bfloat16, per - 1)
    assert CacheManager.pages_within([StateNeed((3,)), None], 4, torch.bfloat16, 100) == 1
    m = CacheManager(needs, 4, CacheManager.pages_within(needs, 4, torch.bfloat16, 3 * per), 2,
                     dtype=torch.bfloat16, allocate=True)
    assert sum(g.storage.numel() * g.storage.element_size() for g in m.groups) == 3 * per


def test_window_group_gives_pages_back_when_the_window_has_passed():
    window = PagedKVNeed(1, 16, window=5)
    m = manager(needs=[FULL, window], page_size=4, num_pages=6)
    full_g, win_g = m.groups
    r = m.open()
    m.reserve(r, 10)
    m.commit(r, 10)        # next query at 10 reads keys 6..10: page 0 (keys 0..3) is dead, page 1 holds 6, 7
    assert r.tables[win_g.index][0] == -1 and r.tables[win_g.index][1] >= 0
    assert all(p >= 0 for p in r.tables[full_g.index])
    assert m.free_pages() == [3, 4]
    m.reserve(r, 3)
    m.commit(r, 3)         # length 13: next query reads 9..13: pages 0, 1 dead
    assert r.tables[win_g.index][:2] == [-1, -1] and len(r.tables[win_g.index]) == 4
    assert m.free_pages() == [2, 4]
    m.audit()
    m.close(r)
    assert m.free_pages() == [6, 6]
    m.audit()


def test_window_one_and_long_run_never_needs_more_than_two_pages():
    m = manager(needs=[PagedKVNeed(1, 16, window=3)], page_size=4, num_pages=3)
    r = m.open()
    for _ in range(200):
        m.reserve(r, 1)
        m.commit(r, 1)
        assert m.used_pages()[0] <= 2
    m.audit()


def test_state_slots_and_zeroing():
    m = CacheManager([[FULL, StateNeed((3,), "float32")], StateNeed((2, 2), "float32")], 4, 4, 2,
                     dtype=torch.float32, device="cpu")
    a, b = m.open(), m.open()
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(OutOfPages):
        m.open()
    m.state[0][a.state_slot] += 7.0
    m.state[1][a.state_slot] += 1.0
    m.close(a)
    c = m.open()
    assert c.state_slot == a.state_slot
    assert float(m.state[0][c.state_slot].abs().sum()) == 0.0 and float(m.state[1][c.state_slot].abs().sum()) == 0.0
    caches = m.layer_caches({0: torch.zeros((1, 1), dtype=torch.int32)})
    assert caches[0].k.shape == (4, 2, 4, 16) and caches[0].state.shape == (2, 3)
    assert caches[1].k is None and caches[1].state.shape == (2, 2, 2)
    m.audit()


def test_misuse_is_caught():
    pool = IdPool(3)
    ids = pool.take(2)
    pool.give(ids)
    with pytest.raises(CacheError, match="twice"):
        pool.give([ids[0]])
    with pytest.raises(CacheError, match="belong"):
        pool.give([17])
    m = manager()
    r = m.open()
    m.reserve(r, 4)
    with pytest.raises(CacheError, match="beyond"):
        m.commit(r, 5)
    m.close(r)
    with pytest.raises(CacheError):
        m.close(r)
    with pytest.raises(CacheError):
        m.reserve(r, 1)
    with pytest.raises(CacheError, match="already open"):
        m.open(rid=5) and m.open(rid=5)


def test_trim_reservation():
    m = manager()
    r = m.open()
    m.reserve(r, 3)
    m.commit(r, 3)
    m.reserve(r, 9)
    assert len(r.tables[0]) == 3
    m.trim_reservation(r)
    assert len(r.tables[0]) == 1 and m.free_pages() == [7]
    m.audit()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    needs = [FULL, PagedKVNeed(2, 16, window=rng.choice([3, 7, 16])), FULL, StateNeed((2,))]
    m = manager(needs=needs, page_size=rng.choice([1, 4, 16]), num_pages=rng.choice([5, 12, 40]), max_requests=4)
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 4:
            live.append(m.open())
        elif op < 0.25 and live:
            m.close(live.pop(rng.randrange(len(live))))
        elif live:
            r = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 17])
            before = [list(t) for t in r.tables]
            free_before = m.free_pages()
            try:
                m.reserve(r, n)
            except OutOfPages:
                assert [list(t) for t in r.tables] == before and m.free_pages() == free_before
                continue
            if rng.random() < 0.9:
                m.commit(r, n)
            else:
                m.trim_reservation(r)
        m.audit()
    for r in live:
        m.close(r)
    m.audit()
    assert all(f == g.pool.n for f, g in zip(m.free_pages(), m.groups))
    assert m.state_slots.free_count == 4

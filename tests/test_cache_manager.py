"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; pages are used again.
(The reference's cache tests: garuda/src/cache/mod.rs:1077-1226.)"""
import random

import numpy as np
import pytest

from garuda_b200.csrc.build import load_host_module

host = load_host_module()


def manager(pages=16, page_size=4, windows=(0,), max_requests=4, max_positions=64):
    return host.CacheManager([host.GroupConfig(pages, w) for w in windows], page_size, max_requests, max_positions)


def test_reserve_commit_release():
    m = manager()
    assert m.acquire(10) == 0 and m.acquire(11) == 1
    m.reserve(10, 9)
    assert list(m.block_table_row(10, 0)[:4]) == [0, 1, 2, -1] and m.free_pages(0) == 13
    m.commit(10, 9)
    assert m.length(10) == 9
    m.reserve(10, 12)                       # still inside the third page
    assert m.free_pages(0) == 13
    m.reserve(10, 13)
    assert m.free_pages(0) == 12
    m.release(10)
    assert m.free_pages(0) == 16 and not m.known(10) and m.free_slots == 3
    m.check_invariants()


def test_pages_come_back_most_recent_first_and_are_used_again():
    m = manager()
    m.acquire(1)
    m.reserve(1, 16)
    m.commit(1, 16)
    first = list(m.block_table_row(1, 0)[:4])
    m.release(1)
    m.acquire(2)
    m.reserve(2, 8)
    again = list(m.block_table_row(2, 0)[:2])
    assert set(again) <= set(first) and m.pages_reused == 2
    m.check_invariants()


def test_all_or_nothing():
    m = manager(pages=4, windows=(0, 0))
    m.acquire(1)
    m.acquire(2)
    m.reserve(1, 12)                        # 3 of 4 pages in both groups
    with pytest.raises(host.OutOfPages):
        m.reserve(2, 8)                     # needs 2
    assert m.free_pages(0) == 1 and m.free_pages(1) == 1
    assert list(m.block_table_row(2, 0)[:2]) == [-1, -1]
    assert not m.can_reserve([(2, 8)]) and m.can_reserve([(2, 4)])
    assert not m.can_reserve([(2, 4), (1, 16)])       # together they need two
    m.check_invariants()


def test_errors():
    m = manager(max_requests=1, max_positions=10)
    m.acquire(1)
    with pytest.raises(host.CacheError, match="already"):
        m.acquire(1)
    with pytest.raises(host.CacheError, match="slot"):
        m.acquire(2)
    with pytest.raises(host.CacheError, match="10-position"):
        m.reserve(1, 11)
    with pytest.raises(host.CacheError, match="backed"):
        m.commit(1, 3)
    with pytest.raises(host.CacheError, match="not known"):
        m.release(99)
    m.release(1)
    with pytest.raises(host.CacheError, match="not known"):
        m.release(1)                        # a second release is refused, not repeated
    m.check_invariants()


def test_window_gives_pages_back_while_running():
    m = manager(pages=6, page_size=4, windows=(0, 6), max_positions=40)
    m.acquire(1)
    n = 0
    for step in (5, 3, 1, 1, 1, 7, 1, 1, 1, 1):
        n += step
        m.reserve(1, n)
        m.commit(1, n)
        m.check_invariants()
        first_live = max(0, n + 1 - 6)      # the next query at position n reads [n+1-6, n]
        assert m.first_live_position(1, n) == first_live
        row = m.block_table_row(1, 1)
        for p in range(len(row)):
            if p < first_live // 4:
                assert row[p] == -1
            elif p < (n + 3) // 4:
                assert row[p] >= 0
        assert all(x >= 0 for x in m.block_table_row(1, 0)[: (n + 3) // 4])
    assert m.free_pages(1) >= 6 - 3         # a window of 6 never holds more than three pages of 4
    m.release(1)
    assert m.free_pages(0) == 6 and m.free_pages(1) == 6


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    windows = rng.choice([(0,), (0, 5), (7, 0, 3)])
    m = manager(pages=rng.choice([6, 10, 24]), page_size=rng.choice([1, 2, 4, 8]), windows=windows,
                max_requests=4, max_positions=48)
    live = {}
    next_id = 1
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and m.free_slots:
            m.acquire(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            want = min(48, live[r] + rng.randint(1, 9))
            if want == live[r]:
                continue
            try:
                m.reserve(r, want)
                m.commit(r, want)
                live[r] = want
            except host.OutOfPages:
                pass
        elif live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        m.check_invariants()
        for r, n in live.items():
            assert m.length(r) == n
    for r in list(live):
        m.release(r)
    m.check_invariants()
    assert all(m.free_pages(g) == m.total_pages(g) for g in range(m.num_groups))
    assert m.free_slots == 4


def test_fill_block_tables():
    m = manager(windows=(0, 3))
    m.acquire(5)
    m.acquire(6)
    m.reserve(5, 6)
    m.reserve(6, 3)
    out = np.full((2, 2, m.max_pages_per_request), 99, dtype=np.int32)
    m.fill_block_tables([6, 5], out)
    assert list(out[0, 0, :2]) == list(m.block_table_row(6, 0)[:2])
    assert list(out[1, 1, :3]) == list(m.block_table_row(5, 1)[:3])
    assert (out[:, :, 2:] == -1).all()

"""The native cache manager: pages, block tables, windows, slots (no GPU)."""
import random

import pytest

from ferrum_b200 import host
from ferrum_b200.errors import CacheError, Unavailable


def manager(groups, max_requests=4):
    h = host.module()
    return h.CacheManager([h.GroupSpec(*g) for g in groups], max_requests)


def test_grow_commit_close_round_trip():
    m = manager([(16, 0, 8, 6)])
    s = m.open()
    assert m.seq_len(s) == 0 and m.pages_missing(s, 33) == [3]
    m.grow(s, 33)
    assert m.pages_held(0, s) == 3 and m.free_pages(0) == 5 and m.seq_len(s) == 0     # grow does not advance
    m.commit(s, 33)
    assert m.seq_len(s) == 33 and m.pages_missing(s, 48) == [0] and m.pages_missing(s, 49) == [1]
    table = m.table(0, s)
    assert len(table) == 6 and sorted(table[:3]) == sorted(set(table[:3])) and table[3:] == [-1, -1, -1]
    m.close(s)
    assert m.free_pages(0) == 8 and m.check() == ""


def test_errors():
    m = manager([(16, 0, 4, 4)], max_requests=2)
    a, b = m.open(), m.open()
    with pytest.raises(Unavailable, match="no free request slots"):      # crates/kvcache/src/pool.rs:83-88
        m.open()
    m.grow(a, 48)
    with pytest.raises(Unavailable, match="no free pages"):
        m.grow(b, 32)
    assert m.pages_held(0, b) == 0                                         # all or nothing
    with pytest.raises(CacheError, match="commit of positions that hold no page"):
        m.commit(b, 5)
    with pytest.raises(CacheError, match="exceeds the block table"):
        m.pages_missing(a, 65)
    m.close(a)
    with pytest.raises(CacheError, match="not open"):                      # crates/kvcache/src/pool.rs:103-112
        m.close(a)
    with pytest.raises(CacheError):
        m.seq_len(a)
    assert m.check() == ""


def test_freed_pages_are_used_again():
    m = manager([(16, 0, 4, 4)])
    a = m.open(); m.grow(a, 64); m.commit(a, 64)
    first = set(m.table(0, a))
    m.close(a)
    b = m.open(); m.grow(b, 64)
    assert set(m.table(0, b)) == first and m.free_pages(0) == 0


def test_window_group_gives_pages_back_as_it_moves():
    """window 20, pages of 8: after n tokens only keys > n - 20 can still be read."""
    m = manager([(8, 20, 10, 64), (8, 0, 64, 64)])
    s = m.open()
    n = 0
    for step in [5, 1, 1, 30, 1, 1, 1, 7, 40, 1]:
        m.grow(s, n + step)
        m.commit(s, n + step)
        n += step
        keep_from = max(0, n - 20 + 1) // 8
        t = m.table(0, s)
        assert all(p < 0 for p in t[:keep_from]) and all(p >= 0 for p in t[keep_from:(n - 1) // 8 + 1])
        assert m.pages_held(1, s) == (n + 7) // 8                         # the full group keeps everything
        assert m.check() == ""
    assert m.pages_held(0, s) <= 4
    with pytest.raises(Unavailable):                                       # a portion larger than the pool
        m.grow(s, n + 80)
    m.close(s)
    assert m.free_pages(0) == 10 and m.free_pages(1) == 64


def test_max_growable():
    m = manager([(16, 0, 5, 16)])
    a, b = m.open(), m.open()
    m.grow(a, 40); m.commit(a, 40)                       # 3 pages
    assert m.max_growable(b, 100) == 32                  # 2 pages left
    assert m.max_growable(a, 100) == 80                  # its own partial page plus 2
    assert m.max_growable(b, 10) == 10


@pytest.mark.parametrize("seed", range(8))
def test_no_page_lost_held_twice_or_freed_twice_under_random_orders(seed):
    rng = random.Random(seed)
    groups = [(16, 0, 24, 12), (8, 24, 10, 24)] if seed % 2 else [(4, 0, 40, 50)]
    m = manager(groups, max_requests=5)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.free_slots():
            live[m.open()] = 0
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            want = live[s] + rng.choice([1, 1, 1, 2, 5, 17, 40])
            cap = min(g[3] * g[0] for g in groups)
            want = min(want, cap)
            if want > live[s] and m.can_grow(s, want):
                m.grow(s, want)
                if rng.random() < 0.9:                   # sometimes the step fails: lengths stay
                    m.commit(s, want)
                    live[s] = want
            elif want > live[s]:
                with pytest.raises(Unavailable):
                    m.grow(s, want)
        elif live:
            s = rng.choice(list(live))
            m.close(s)
            del live[s]
        assert m.check() == "", m.check()
        held = [set(p for p in m.table(g, s) if p >= 0) for g in range(len(groups)) for s in live]
        for g in range(len(groups)):
            pages = [p for s in live for p in m.table(g, s) if p >= 0]
            assert len(pages) == len(set(pages)) == m.used_pages(g)
    for s in list(live):
        m.close(s)
    assert all(m.free_pages(g) == groups[g][2] for g in range(len(groups))) and m.check() == ""


def test_the_page_reuse_check_of_the_gpu_tests_can_fail():
    """The GPU tests assert that some page was held by two requests (helpers.pages_were_reused).
    Here the same bookkeeping on the manager alone: true when a closed request's pages go to the
    next one, false when the pool is so large that nothing is ever handed out twice."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import pages_were_reused, record_owners
    for pool, close_first, expect in ((4, True, True), (8, False, False)):
        m = manager([(16, 0, pool, 4)])
        owners, slots = {}, {}
        slots["a"] = m.open()
        m.grow(slots["a"], 40)
        record_owners(owners, m, slots)
        if close_first:
            m.close(slots.pop("a"))
        slots["b"] = m.open()
        m.grow(slots["b"], 40)
        record_owners(owners, m, slots)
        assert pages_were_reused(owners) is expect

"""The cache's bookkeeping on the host: no slot or page is lost, held twice or
freed twice; a window group gives back the pages its queries have passed."""
import random

import pytest
import torch

from janus_b200.cache import PAGE_SIZE, CacheFull, PagePool, SequenceCache
from janus_b200.parts.base import KVSpec, StateSpec

CPU = torch.device("cpu")


def test_page_pool_take_and_give_back():
    pool = PagePool(4)
    got = [pool.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and pool.n_free == 0
    with pytest.raises(CacheFull):
        pool.take()
    pool.give_back(got[1])
    with pytest.raises(ValueError, match="not held"):
        pool.give_back(got[1])                     # freed twice
    with pytest.raises(ValueError):
        pool.give_back(99)
    assert pool.take() == got[1]
    pool.check()


def make_cache(max_tokens=PAGE_SIZE * 6, n_slots=3, window=0):
    specs = [KVSpec(2, 16), KVSpec(2, 16), None, StateSpec((5,))]
    if window:
        specs.append(KVSpec(2, 16, window))
    return SequenceCache(specs, max_tokens, n_slots, torch.float32, CPU)


def test_groups_and_storage():
    c = make_cache(window=100)
    assert len(c.groups) == 2                                   # all-keys layers and window layers apart
    full, win = c.groups
    assert full.places == [0, 1] and win.places == [4]
    assert full.k[0].shape == (6, 2, PAGE_SIZE, 16) and 2 not in c.group_of_place
    assert c.states[3].shape == (3, 5)


def test_slots_are_reused_and_state_is_zeroed():
    c = make_cache()
    a, b, d = c.alloc_slot(), c.alloc_slot(), c.alloc_slot()
    assert sorted((a, b, d)) == [0, 1, 2]
    with pytest.raises(CacheFull):
        c.alloc_slot()
    c.states[3][b] = 7.0
    c.free_slot(b)
    with pytest.raises(ValueError):
        c.free_slot(b)                              # freed twice
    with pytest.raises(ValueError):
        c.length(b)
    again = c.alloc_slot()
    assert again == b and float(c.states[3][again].abs().sum()) == 0.0 and c.length(again) == 0
    c.check()


def test_reserve_advance_and_full():
    c = make_cache()
    s, t = c.alloc_slot(), c.alloc_slot()
    c.reserve(s, 70)
    c.advance(s, 70)
    assert c.length(s) == 70 and len(c.groups[0].pages[s]) == 2
    rows = c.groups[0].dest_rows(s, 60, 10)
    p0, p1 = c.groups[0].pages[s]
    assert rows.tolist() == [p0 * PAGE_SIZE + r for r in range(60, 64)] + [p1 * PAGE_SIZE + r for r in range(6)]
    c.reserve(t, PAGE_SIZE * 4)
    with pytest.raises(CacheFull):
        c.reserve(s, PAGE_SIZE)                    # 2 + 4 pages held, a seventh is needed
    assert len(c.groups[0].pages[s]) == 2          # the failed call changed nothing
    c.check()
    c.free_slot(t)
    c.reserve(s, PAGE_SIZE)
    c.check()


def test_window_group_gives_back_passed_pages():
    w = 70
    c = SequenceCache([KVSpec(1, 8, w)], PAGE_SIZE * 4, 2, torch.float32, CPU)
    s = c.alloc_slot()
    g = c.groups[0]
    total = 0
    for n in (100, 1, 1, 60, 1, 30, 1, 1):
        c.reserve(s, n)
        c.advance(s, n)
        total += n
        first_needed = max(0, total - w + 1)
        for i, p in enumerate(g.pages[s]):
            assert (p == -1) == ((i + 1) * PAGE_SIZE <= first_needed), (total, i, p)
        c.check()
    assert g.pool.n_held <= (w + PAGE_SIZE - 1) // PAGE_SIZE + 1
    c.free_slot(s)
    assert g.pool.n_held == 0


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make_cache(max_tokens=PAGE_SIZE * 12, n_slots=4, window=90)
    live = {}
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and c.n_free_slots:
            live[c.alloc_slot()] = 0
        elif r < 0.4 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 17, 64, 130])
            try:
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            except CacheFull:
                pass
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pool.n_held == 0 for g in c.groups) and c.n_free_slots == 4

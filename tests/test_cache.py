"""The cache's bookkeeping on the host: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import numpy as np
import pytest
import torch

from ember_cpp_b200.cache import PAGE, CacheError, Pool, PoolError, SequenceCache
from ember_cpp_b200.parts import CacheNeed, StateNeed

FULL = CacheNeed("full", 2, 16)
WIN = CacheNeed("window", 1, 32, window=70)


def make(needs=((FULL, None),), cache_of=None, max_tokens=512, max_positions=None, max_slots=None):
    needs = list(needs)
    return SequenceCache(needs, cache_of or [None] * len(needs), max_tokens, max_positions, torch.float32, "cpu", max_slots)


def test_pool_take_give_back():
    p = Pool(3, "slot")
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.free == 0
    with pytest.raises(PoolError, match="no free slot"):
        p.take()
    p.give_back(b)
    with pytest.raises(PoolError, match="not held"):
        p.give_back(b)
    with pytest.raises(PoolError, match="does not exist"):
        p.give_back(7)
    assert p.take() == b          # the unit given back last is used again first
    p.check()


def test_sizes_follow_max_tokens():
    c = make(max_tokens=1000, max_positions=200)
    assert c.n_pages == 16 and c.max_tokens == 1024 and c.n_slots == 16
    assert c.max_blocks == 4      # 200 positions round up to 4 pages
    assert tuple(c.groups[0].k[0].shape) == (16, 2, PAGE, 16)
    with pytest.raises(CacheError):
        make(max_tokens=0)


def test_groups_have_storage_of_their_own():
    c = make(needs=[(FULL, None), (WIN, None), (FULL, None), (WIN, None), (FULL, None)],
             cache_of=[None, None, None, None, 0])
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.apps == [0, 2] and win.apps == [1, 3]            # the sharing entry has no storage
    assert c.views[4] is c.views[0] and c.writes == [True, True, True, True, False]
    assert c.views[1].window == 70 and c.views[0].window == 0
    assert c.views[0].k.data_ptr() != c.views[2].k.data_ptr()
    assert tuple(win.k[0].shape) == (8, 1, PAGE, 32)


def test_reserve_is_all_or_nothing():
    c = make(max_tokens=256)                  # 4 pages
    a, b = c.open(), c.open()
    c.reserve([(a, 100), (b, 60)])            # 2 + 1 pages
    c.commit([(a, 100), (b, 60)])
    before = [list(h) for h in c.groups[0].held]
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve([(a, 1), (b, 70)])          # b would need 2 more pages, 1 is free
    assert [list(h) for h in c.groups[0].held] == before and c.groups[0].pages.free == 1
    with pytest.raises(CacheError, match="twice"):
        c.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="not open"):
        c.reserve([(3, 1)])
    c.check()


def test_positions_bounded_by_the_model():
    c = make(max_tokens=512, max_positions=100)
    s = c.open()
    with pytest.raises(CacheError, match="100 positions"):
        c.reserve([(s, 101)])
    c.reserve([(s, 100)])
    c.commit([(s, 100)])
    with pytest.raises(CacheError, match="exceeds"):
        c.reserve([(s, 1)])


def test_close_gives_everything_back_and_slots_are_reused():
    c = make(max_tokens=256)
    a = c.open()
    c.reserve([(a, 200)])
    c.commit([(a, 200)])
    assert c.groups[0].pages.free == 0
    c.close(a)
    assert c.groups[0].pages.free == 4 and c.slots.free == 4
    with pytest.raises(CacheError, match="not open"):
        c.close(a)
    assert c.open() == a and c.length(a) == 0
    c.check()


def test_window_group_gives_back_old_pages():
    c = make(needs=[(FULL, None), (WIN, None)], max_tokens=1024)
    full, win = c.groups
    s = c.open()
    c.reserve([(s, 200)])                     # a prompt needs all its pages during the step
    assert sum(p >= 0 for p in win.held[s]) == 4
    c.commit([(s, 200)])                      # next query at 200 reads 131..200: blocks 2, 3
    assert [p >= 0 for p in win.held[s]] == [False, False, True, True]
    assert sum(p >= 0 for p in full.held[s]) == 4
    for _ in range(120):                      # decode on: the window slides, pages come and go
        n = c.length(s)
        c.reserve([(s, 1)])
        c.commit([(s, 1)])
        first = max(0, n + 1 - 70 + 1) // PAGE
        held = [i for i, p in enumerate(win.held[s]) if p >= 0]
        assert held == list(range(first, -(-(n + 1) // PAGE)))
        c.check()
    table = win.table([s, -1], 8)
    assert table.shape == (2, 8) and (table[1] == -1).all() and (table[0, :first] == -1).all()
    c.close(s)
    assert win.pages.free == win.pages.size and full.pages.free == full.pages.size


def test_state_rows_are_reset_when_a_slot_opens():
    c = make(needs=[(FULL, StateNeed((3, 2), init=0.5)), (FULL, None)], max_tokens=128)
    assert c.states[1] is None and tuple(c.states[0].shape) == (2, 3, 2)
    s = c.open()
    c.states[0][s] += 1.0
    c.close(s)
    assert c.open() == s and torch.all(c.states[0][s] == 0.5)


def test_truncate():
    c = make(max_tokens=512)
    s = c.open()
    c.reserve([(s, 130)])
    c.commit([(s, 130)])
    c.truncate(s, 64)
    assert c.length(s) == 64 and len(c.groups[0].held[s]) == 1
    with pytest.raises(CacheError):
        c.truncate(s, 65)
    c.check()


def test_random_traffic_keeps_the_books():
    rnd = random.Random(0)
    c = make(needs=[(FULL, None), (WIN, None)], max_tokens=64 * 24, max_positions=400, max_slots=6)
    live = []
    for _ in range(600):
        op = rnd.random()
        if op < 0.25 and c.slots.free:
            live.append(c.open())
        elif op < 0.4 and live:
            c.close(live.pop(rnd.randrange(len(live))))
        elif live:
            batch = rnd.sample(live, rnd.randint(1, len(live)))
            step = [(s, rnd.choice([1, 1, 1, 5, 64, 130]) if c.length(s) else rnd.randint(1, 200)) for s in batch]
            try:
                c.reserve(step)
            except CacheError:
                c.check()
                continue
            c.commit(step)
            for s, _ in step:
                for g in c.groups:
                    need = range(g.first_needed_block(c.length(s)), -(-c.length(s) // PAGE))
                    assert all(g.held[s][b] >= 0 for b in need)
        c.check()
    for s in live:
        c.close(s)
    c.check()
    assert all(g.pages.free == g.pages.size for g in c.groups) and c.slots.free == c.n_slots


def test_tails_of_new_pages_are_named_for_clearing():
    """`reserve` names, per group and sequence, the rows past the step's end in a page that is new to
    the sequence: those rows hold what the page's last owner left and the step does not write them."""
    c = make(max_tokens=64 * 8)
    a, b = c.open(), c.open()
    tails = c.reserve([(a, 70), (b, 64)])                 # a: pages 0 and 1, ends at row 6 of page 1; b: one full page
    page_a1 = c.groups[0].held[a][1]
    assert tails == [[(page_a1, 6), (-1, 0)]]
    c.commit([(a, 70), (b, 64)])
    tails = c.reserve([(a, 1), (b, 1)])                   # a stays in its page; b takes a new page and writes row 0
    assert tails == [[(-1, 0), (c.groups[0].held[b][1], 1)]]
    c.commit([(a, 1), (b, 1)])
    tails = c.reserve([(a, 57), (b, 63)])                 # both end exactly at a page's edge: nothing to clear
    assert tails == [[(-1, 0), (-1, 0)]]
    c.commit([(a, 57), (b, 63)])
    c.check()

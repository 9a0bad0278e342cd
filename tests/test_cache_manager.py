"""The cache manager on the CPU: no page lost, held twice or freed twice under random orders of
requests; windows give pages back; groups have pages of their own; state slots are zeroed."""
from __future__ import annotations

import random

import pytest
import torch

from stride_b200.cache.manager import NO_PAGE, CacheError, CacheManager
from stride_b200.parts import CacheNeed


def _needs(window=0):
    full = CacheNeed("pages", kv_heads=2, head_dim=4, window=0, dtype=torch.float32)
    win = CacheNeed("pages", kv_heads=2, head_dim=4, window=window, dtype=torch.float32)
    state = CacheNeed("state", state_shape=(3,), state_dtype=torch.float32)
    return [full, win if window else full, state, ("shared", 0), None, full]


def test_groups_slots_and_views():
    cm = CacheManager(_needs(window=10), device="cpu", max_slots=3, max_context=64, page_size=4, num_pages=12)
    assert len(cm.groups) == 2 and cm.groups[0].entries == [0, 5] and cm.groups[1].entries == [1]
    assert cm.groups[0].arena.shape == (13, 2, 2, 2, 4, 4)      # one spare page for padding rows
    a, b = cm.layer_cache(0), cm.layer_cache(3)
    assert b.pages.data_ptr() == a.pages.data_ptr() and a.writes and not b.writes
    assert cm.layer_cache(5).pages.data_ptr() != a.pages.data_ptr()
    assert cm.layer_cache(2).state.shape == (4, 3) and cm.layer_cache(4).pages is None
    s = cm.acquire_slot()
    cm.layer_cache(2).state[s] += 5
    cm.release_slot(s)
    assert cm.acquire_slot() == s and float(cm.layer_cache(2).state[s].abs().sum()) == 0   # zeroed on acquire
    assert [cm.acquire_slot(), cm.acquire_slot(), cm.acquire_slot()] == [1, 2, -1]


def test_ensure_is_all_or_nothing_and_pages_are_reused():
    cm = CacheManager(_needs(), device="cpu", max_slots=4, max_context=64, page_size=4, num_pages=6)
    a, b = cm.acquire_slot(), cm.acquire_slot()
    assert cm.pages_needed(a, 9) == [3] and cm.ensure(a, 9) and cm.free_pages() == [3]
    assert cm.pages_needed(a, 12) == [0] and cm.pages_needed(a, 13) == [1]
    assert not cm.ensure(b, 17) and cm.free_pages() == [3] and cm.length[b] == 0    # refused, nothing changed
    assert cm.ensure(b, 12) and cm.free_pages() == [0]
    held_a = set(cm.groups[0].held[a].values())
    cm.release_slot(a)
    c = cm.acquire_slot()
    assert cm.ensure(c, 10) and set(cm.groups[0].held[c].values()) == held_a          # the same pages again
    assert (cm.groups[0].table_host[a] == NO_PAGE).sum() == cm.max_pages_per_seq - 3
    cm.check()
    with pytest.raises(CacheError, match="exceeds the context capacity"):
        cm.ensure(c, 65)
    cm.release_slot(b)
    with pytest.raises(CacheError, match="released but not held"):
        cm.release_slot(b)


def test_window_gives_pages_back():
    cm = CacheManager(_needs(window=6), device="cpu", max_slots=2, max_context=200, page_size=4, num_pages=50)
    s = cm.acquire_slot()
    for n in range(1, 101):
        assert cm.ensure(s, n)
        cm.trim(s)
        kept = cm.groups[1].held[s]
        first_needed = n - 6 + 1                       # the oldest key the next token reads
        assert all((i + 1) * 4 > first_needed for i in kept)
        assert all(i in kept for i in range(max(0, first_needed) // 4, (n - 1) // 4 + 1))
        assert len(kept) <= 3
    assert len(cm.groups[0].held[s]) == 25             # the group without a window keeps everything
    cm.check()
    # a portion longer than the window: all its pages are there while it runs, then most go back
    t = cm.acquire_slot()
    assert cm.ensure(t, 40) and len(cm.groups[1].held[t]) == 10
    assert cm.trim(t) == 8
    cm.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    cm = CacheManager(_needs(window=rng.choice([0, 5, 9])), device="cpu", max_slots=5, max_context=48, page_size=rng.choice([2, 4, 8]),
                      num_pages=rng.choice([7, 15, 40]), shuffle_seed=seed)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 5:
            s = cm.acquire_slot()
            assert s >= 0 and s not in live
            live[s] = 0
        elif op < 0.75 and live:
            s = rng.choice(list(live))
            end = min(48, live[s] + rng.randint(1, 9))
            need, free = cm.pages_needed(s, end), cm.free_pages()
            ok = cm.ensure(s, end)
            assert ok == all(n <= f for n, f in zip(need, free))
            if ok:
                assert cm.free_pages() == [f - n for n, f in zip(need, free)]
                live[s] = max(live[s], end)
                if rng.random() < 0.7:
                    cm.trim(s)
        elif live:
            s = rng.choice(list(live))
            cm.release_slot(s)
            del live[s]
        cm.check()
    for s in list(live):
        cm.release_slot(s)
    cm.check()
    assert cm.free_pages() == cm.total_pages() and len(cm.free_slots) == 5


def test_check_finds_damaged_books():
    cm = CacheManager(_needs(), device="cpu", max_slots=3, max_context=64, page_size=4, num_pages=8)
    a, b = cm.acquire_slot(), cm.acquire_slot()
    assert cm.ensure(a, 8) and cm.ensure(b, 8)
    cm.check()
    table = cm.groups[0].table_host
    mine = int(table[b, 0])
    table[b, 0] = table[a, 0]
    with pytest.raises(CacheError, match="is also held by slot"):
        cm.check()
    table[b, 0] = NO_PAGE
    with pytest.raises(CacheError, match="but 2 are counted"):
        cm.check()
    table[b, 0] = mine
    cm.check()
    table[2, 0] = 7                                    # a slot nobody holds
    with pytest.raises(CacheError, match="not live"):
        cm.check()

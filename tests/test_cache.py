"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from minfer_b200.cache.paged import (PAGE, Cache, CacheError, GroupKey, OutOfPages, PagePool,
                                     SlotTable, pages_for)


def _cache(max_tokens=1024, max_seqs=4):
    reqs = {0: GroupKey(2, 16, 0), 1: GroupKey(2, 16, 70), 2: GroupKey(2, 16, 70),
            3: GroupKey(1, 32, 0)}
    return Cache(reqs, max_tokens, max_seqs, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.groups) == 3
    g_lin, g_win, g_other = c.group_of[0], c.group_of[1], c.group_of[3]
    assert c.group_of[2] is g_win and g_lin is not g_win and g_other is not g_lin
    # 16 pages the pool hands out plus the spare page that only padding rows of a batch touch
    assert g_lin.k.shape == (1, 16 + 1, 2, PAGE, 16) and g_win.k.shape[0] == 2
    assert g_lin.spare_page == 16 and g_lin.pool.n_free() == 16
    assert g_lin.table_rows([c.spare_slot], 3) == [[16, -1, -1]]
    assert g_win.ring == 128 and g_lin.ring == 0
    assert g_win.n_pages == min(16, 4 * 2)


def test_slots_are_unique_and_cannot_be_freed_twice():
    t = SlotTable(3)
    a, b, c = t.acquire(), t.acquire(), t.acquire()
    assert len({a, b, c}) == 3
    with pytest.raises(CacheError, match="in use"):
        t.acquire()
    t.release(b)
    with pytest.raises(CacheError, match="released twice"):
        t.release(b)
    with pytest.raises(CacheError, match="out of range"):
        t.release(7)
    assert t.acquire() == b


def test_pages_follow_length_and_rings_stop_growing():
    c = _cache()
    s = c.acquire()
    c.reserve(s, 1)
    assert [len(g.pages[s]) for g in c.groups] == [1, 1, 1]
    c.reserve(s, 65)
    assert [len(g.pages[s]) for g in c.groups] == [2, 2, 2]
    c.reserve(s, 300)
    assert len(c.group_of[0].pages[s]) == pages_for(300) and len(c.group_of[1].pages[s]) == 2
    c.release(s)
    assert c.free_pages() == [g.n_pages for g in c.groups]
    with pytest.raises(CacheError):
        c.reserve(s, 10)                    # the slot is no longer held


def test_running_out_of_pages_is_an_error():
    c = _cache(max_tokens=128, max_seqs=2)
    s = c.acquire()
    with pytest.raises(OutOfPages, match="no free page"):
        c.reserve(s, 129)


def test_a_page_is_never_held_twice_nor_lost_under_churn():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 40, max_seqs=6)
    live = {}
    for _ in range(600):
        if live and (rng.random() < 0.3 or len(live) == 6):
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif len(live) < 6 and rng.random() < 0.5:
            live[c.acquire()] = 0
        elif live:
            s = rng.choice(list(live))
            grow = live[s] + rng.randint(1, 90)
            try:
                c.reserve(s, grow)
                c.set_length(s, grow)
                live[s] = grow
            except OutOfPages:
                pass
        for g in c.groups:
            held = [p for s in range(6) for p in g.pages[s]]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + g.pool.n_free() == g.n_pages, "a page was lost"
            for s in range(6):
                assert all(g.pool.owner(p) == s for p in g.pages[s])
                if s not in live:
                    assert g.pages[s] == []
            # the integer table a step's page tables are cut from mirrors the page lists
            rows = list(live) + [c.spare_slot]
            width = max(1, g.max_pages_of(rows)) + rng.randint(0, 2)
            assert g.table_flat(rows, width) == [p for r in g.table_rows(rows, width) for p in r]
    for s in list(live):
        c.release(s)
    assert c.free_pages() == [g.n_pages for g in c.groups]
    assert c.slots.n_free() == 6


def test_giving_back_a_page_twice_is_refused():
    p = PagePool(4)
    a = p.take(0)
    p.give_back(a, 0)
    with pytest.raises(CacheError, match="held by"):
        p.give_back(a, 0)


def test_state_is_zeroed_when_a_slot_is_handed_out():
    c = _cache()
    t = c.state.add("memory", (3,), torch.float32)
    s = c.acquire()
    t[s] = 5.0
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(t[s2].abs().sum()) == 0.0
    assert c.state.bytes_per_slot() == 12


def test_guards_around_storage():
    """The bytes before and after a tensor hold a fixed value; changing one is seen."""
    import torch
    from minfer_b200.cache.paged import Cache, CacheError, GroupKey, Guarded
    g = Guarded((3, 5), torch.float32, "cpu", "a test tensor")
    assert g.tensor.shape == (3, 5) and float(g.tensor.abs().sum()) == 0.0
    g.tensor.fill_(7.0)                                 # writing the tensor itself is fine
    assert g.intact()
    g.raw[255] = 0
    assert not g.intact()
    cache = Cache({0: GroupKey(2, 16, 0), 1: GroupKey(2, 16, 40)}, 256, 2, torch.float32, "cpu")
    cache.state.add("x", (4,), torch.int32)
    cache.check_canaries()
    cache.groups[1]._guarded[0].raw[-1] = 1
    try:
        cache.check_canaries()
        raise AssertionError("a changed guard was not seen")
    except CacheError as e:
        assert "keys of cache group" in str(e)

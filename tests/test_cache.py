"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""

import random

import pytest
import torch

from enginekernel_b200.cache import PAGE, CacheError, FreeList, PageGroup, SequenceCache, SlotBook
from enginekernel_b200.parts.spec import CacheSpec


def test_free_list_refuses_double_free_and_exhaustion():
    f = FreeList(3, "thing")
    a, b, c = f.take(), f.take(), f.take()
    assert sorted((a, b, c)) == [0, 1, 2]
    with pytest.raises(CacheError, match="no free thing"):
        f.take()
    f.give_back(b)
    with pytest.raises(CacheError, match="not held"):
        f.give_back(b)
    with pytest.raises(CacheError, match="does not exist"):
        f.give_back(7)
    assert f.take() == b and f.available() == 0


def make_cache(max_tokens=640, slots=4, window=None, max_len=None):
    specs = [CacheSpec("kv", heads=2, head_dim=16), CacheSpec("kv", heads=2, head_dim=16),
             CacheSpec("kv", heads=2, head_dim=16, window=window) if window else None,
             CacheSpec("state", shape=(3, 2))]
    return SequenceCache(specs, torch.float32, "cpu", max_tokens=max_tokens, max_slots=slots,
                         max_len=max_len)


def test_pages_follow_lengths_and_come_back():
    c = make_cache()
    assert c.num_pages == 10 and c.free_tokens() == 640
    s = c.open()
    c.reserve(s, 1)
    assert c.free_tokens() == 640 - PAGE
    c.reserve(s, 64)                        # still the same page
    assert c.free_tokens() == 640 - PAGE
    c.reserve(s, 65)
    assert c.free_tokens() == 640 - 2 * PAGE
    c.advance(s, 65)
    assert c.length(s) == 65
    t = c.open()
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve(t, 9 * PAGE)              # 8 pages are left
    assert c.free_tokens() == 640 - 2 * PAGE   # a refused reservation takes nothing
    c.reserve(t, 8 * PAGE)
    assert c.free_tokens() == 0
    c.close(s)
    assert c.free_tokens() == 2 * PAGE
    with pytest.raises(CacheError, match="not open"):
        c.close(s)
    with pytest.raises(CacheError, match="not open"):
        c.reserve(s, 5)
    with pytest.raises(CacheError, match="not open"):
        c.length(s)
    c.close(t)
    assert c.free_tokens() == 640 and c.book.open_slots() == []


def test_slots_run_out_and_are_used_again():
    c = make_cache(slots=2)
    a, b = c.open(), c.open()
    with pytest.raises(CacheError, match="no free sequence slot"):
        c.open()
    c.close(a)
    again = c.open()
    assert again == a and c.length(again) == 0 and c.book.generation[a] == 2


def test_length_limit():
    c = make_cache(max_tokens=640, max_len=100)
    s = c.open()
    with pytest.raises(CacheError, match="limit"):
        c.reserve(s, 101)
    c.reserve(s, 100)


def test_state_is_zeroed_when_a_slot_is_taken():
    c = make_cache()
    s = c.open()
    c.entry(3).state[s] = 5.0
    c.close(s)
    assert c.open() == s
    assert c.entry(3).state[s].abs().sum().item() == 0
    assert c.entry(3).state.shape == (c.num_slots, 3, 2)
    assert c.entry(0).k_pages.shape == (c.num_pages, 2, PAGE, 16)
    assert c.entry(0).k_pages.data_ptr() != c.entry(1).k_pages.data_ptr()
    with pytest.raises(CacheError):
        c.entry(2)                          # no window group was asked for here


def test_groups_have_storage_of_their_own_and_windows_give_pages_back():
    c = make_cache(max_tokens=64 * 20, window=100)
    full = c.entry(0)._group.page_group
    win = c.entry(2)._group.page_group
    assert full is not win and full is c.entry(1)._group.page_group
    s = c.open()
    c.reserve(s, 300)
    c.advance(s, 300)
    # the next token (position 300) reads keys 201..300: logical pages 3 and 4 remain
    assert len(full.pages_of(s)) == 5 and len(win.pages_of(s)) == 2
    assert win.table[s][:3] == [-1, -1, -1] and win.table[s][3] >= 0
    for n in range(301, 400):
        c.reserve(s, n)
        c.advance(s, 1)
        assert len(win.pages_of(s)) <= 3
    c.close(s)
    assert full.pool.available() == 20 and win.pool.available() == 20


def test_block_table_upload_matches_host_table():
    c = make_cache()
    a, b = c.open(), c.open()
    c.reserve(a, 130)
    c.reserve(b, 10)
    c.upload_tables()
    g = c.entry(0)._group
    assert g.block_table[a, :3].tolist() == g.page_group.table[a][:3]
    assert g.block_table[b, 0].item() == g.page_group.table[b][0]
    assert not g.page_group.dirty


def test_random_churn_never_loses_or_doubles_a_page():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 40, slots=6, window=70)
    groups = [g.page_group for g in c.groups if g.page_group is not None]
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            live[c.open()] = 0
        elif op < 0.4 and live:
            s = rng.choice(list(live))
            c.close(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 5, 64, 90])
            try:
                c.reserve(s, live[s] + n)
            except CacheError:
                continue
            c.advance(s, n)
            live[s] += n
        for g in groups:
            held = [p for s in range(c.num_slots) for p in g.table[s] if p >= 0]
            assert len(held) == len(set(held))                          # none held twice
            assert len(held) + g.pool.available() == g.pool.n           # none lost
            assert sorted(held) == g.pool.held()
        assert sorted(live) == c.book.open_slots()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.close(s)
    assert all(g.pool.available() == g.pool.n for g in groups)


def test_a_step_of_several_sequences_gets_all_its_pages_or_none():
    """Three sequences ask together for more pages than are left: none of them keeps a page, and
    what was free before is free after (a step that cannot run must not shrink the cache)."""
    c = make_cache()                                    # 10 pages
    a, b, d = c.open(), c.open(), c.open()
    c.reserve(a, 2 * PAGE)
    c.advance(a, 2 * PAGE)
    before = c.free_tokens()
    assert before == 8 * PAGE
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve_all([(a, 5 * PAGE), (b, 3 * PAGE), (d, 3 * PAGE + 1)])      # 3 + 3 + 4 = 10 > 8
    assert c.free_tokens() == before
    for g in c.groups:
        if g.page_group is not None:
            assert g.page_group.pages_of(b) == [] and g.page_group.pages_of(d) == []
            assert len(g.page_group.pages_of(a)) == 2
    c.reserve_all([(a, 5 * PAGE), (b, 3 * PAGE), (d, 2 * PAGE)])              # 3 + 3 + 2 = 8
    assert c.free_tokens() == 0
    with pytest.raises(CacheError, match="not open"):
        c.reserve_all([(a, 5 * PAGE), (3, 1)])
    for s in (a, b, d):
        c.close(s)
    assert c.free_tokens() == 10 * PAGE

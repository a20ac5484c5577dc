"""The cache's bookkeeping (no GPU): no page or slot is lost, held twice or freed twice."""

import random

import numpy as np
import pytest
import torch

from rusty_llama_b200.cache import PAGE_SIZE, Cache, PagePool
from rusty_llama_b200.errors import CacheError
from rusty_llama_b200.parts import KVNeed, StateNeed


def make_cache(max_tokens=64 * 8, max_seqs=4, window=0, with_state=True):
    needs = [(0, KVNeed(2, 16, 0)), (1, KVNeed(2, 16, 0)), (2, KVNeed(2, 16, window or 0))]
    if window:
        needs[2] = (2, KVNeed(2, 16, window))
    if with_state:
        needs.append((3, StateNeed((5,), torch.float32)))
    return Cache(needs, max_tokens, max_seqs, torch.float32, "cpu")


def test_page_pool_refuses_double_free_and_exhaustion():
    p = PagePool(3)
    pages = [p.take() for _ in range(3)]
    assert sorted(pages) == [0, 1, 2] and p.n_free == 0
    with pytest.raises(CacheError, match="out of cache pages"):
        p.take()
    p.give_back(pages[1])
    with pytest.raises(CacheError, match="twice"):
        p.give_back(pages[1])
    with pytest.raises(CacheError, match="does not exist"):
        p.give_back(7)
    assert p.take() == pages[1]


def test_groups_are_formed_by_need():
    c = make_cache(window=100)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    assert c.kv_groups[0].runs == [0, 1] and c.kv_groups[1].runs == [2]
    assert c.kv_groups[0].k.shape == (2, 8, 2, PAGE_SIZE, 16)
    assert c.where(1) == ("kv", 0, 1) and c.where(3) == ("state", 0, 0)
    with pytest.raises(CacheError, match="owns no cache"):
        c.where(9)
    assert c.view(1).k_pages.data_ptr() == c.kv_groups[0].k[1].data_ptr()


def test_slots_are_reused_and_not_freed_twice():
    c = make_cache()
    a, b = c.open_sequence(), c.open_sequence()
    assert {a, b} == {0, 1}
    c.close_sequence(a)
    with pytest.raises(CacheError, match="not open"):
        c.close_sequence(a)
    with pytest.raises(CacheError, match="not open"):
        c.length(a)
    assert c.open_sequence() == a  # the freed slot is used again
    for _ in range(2):
        c.open_sequence()
    with pytest.raises(CacheError, match="all 4 sequence slots"):
        c.open_sequence()
    c.check_consistent()


def test_reserve_is_all_or_nothing():
    c = make_cache(max_tokens=64 * 4)
    a, b = c.open_sequence(), c.open_sequence()
    c.reserve([a], [100])  # 2 pages
    c.commit([a], [100])
    free_before = c.pages_free()
    with pytest.raises(CacheError, match="out of cache pages"):
        c.reserve([a, b], [30, 200])  # a needs 1 more, b needs 4: does not fit
    assert c.pages_free() == free_before
    c.check_consistent()
    with pytest.raises(CacheError, match="twice"):
        c.reserve([a, a], [1, 1])
    c.reserve([a, b], [28, 64])
    c.commit([a, b], [28, 64])
    assert c.length(a) == 128 and c.length(b) == 64 and c.pages_free() == 1
    c.close_sequence(a)
    assert c.pages_free() == 3
    c.check_consistent()


def test_state_is_zeroed_when_a_slot_opens():
    c = make_cache()
    a = c.open_sequence()
    view = c.view(3)
    view.state[a] += 7.0
    c.close_sequence(a)
    assert c.open_sequence() == a
    assert (c.view(3).state[a] == 0).all()


def test_window_group_gives_pages_back():
    c = make_cache(max_tokens=64 * 16, window=100)
    a = c.open_sequence()
    full, win = c.kv_groups[0], c.kv_groups[1]
    for step_len in [200] + [1] * 300:
        c.reserve([a], [step_len])
        c.commit([a], [step_len])
        c.check_consistent()
    n = c.length(a)
    assert n == 500
    assert sum(p >= 0 for p in full.pages[a]) == (n + 63) // 64
    held = [i for i, p in enumerate(win.pages[a]) if p >= 0]
    assert held[0] == (n - 100 + 1) // 64 and held[-1] == (n - 1) // 64
    # the table shows 0 for pages that were given back
    t = c.block_table(1, [a], c.table_width([a]))
    assert (t[0, : held[0]] == 0).all()
    c.close_sequence(a)
    assert full.pool.n_free == 16 and win.pool.n_free == 16


def test_random_traffic_keeps_every_page_accounted_for():
    rnd = random.Random(0)
    c = make_cache(max_tokens=64 * 24, max_seqs=6, window=70)
    live = {}
    for _ in range(600):
        op = rnd.random()
        if op < 0.25 and len(live) < 6:
            live[c.open_sequence()] = 0
        elif op < 0.4 and live:
            s = rnd.choice(list(live))
            c.close_sequence(s)
            del live[s]
        elif live:
            k = rnd.randint(1, len(live))
            slots = rnd.sample(list(live), k)
            lens = [rnd.choice([1, 1, 1, 5, 64, 130]) for _ in slots]
            try:
                c.reserve(slots, lens)
            except CacheError:
                c.check_consistent()
                continue
            c.commit(slots, lens)
            for s, q in zip(slots, lens):
                live[s] += q
        c.check_consistent()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.close_sequence(s)
    c.check_consistent()
    assert all(g.pool.n_free == g.pool.n_pages for g in c.kv_groups) and c.n_open == 0


def test_block_table_lists_pages_in_position_order():
    c = make_cache()
    a, b = c.open_sequence(), c.open_sequence()
    c.reserve([a, b], [65, 10])
    c.commit([a, b], [65, 10])
    t = c.block_table(0, [b, a], 4)
    assert t.dtype == np.int32 and t.shape == (2, 4)
    assert list(t[1, :2]) == c.kv_groups[0].pages[a] and t[0, 0] == c.kv_groups[0].pages[b][0]
    assert len(set(c.kv_groups[0].pages[a]) | set(c.kv_groups[0].pages[b])) == 3


def test_workspace_keeps_what_replayed_graphs_may_still_write_to():
    """A scratch tensor that has to grow is replaced, never freed: a graph captured earlier still uses
    the old address.  Zeroed tensors start as zeros."""
    from rusty_llama_b200.parts import Workspace

    ws = Workspace(torch.device("cpu"))
    a = ws.get("scratch", 10, torch.float32)
    assert ws.get("scratch", 8, torch.float32) is a  # large enough: the same tensor
    ptr = a.data_ptr()
    del a
    b = ws.get("scratch", 1000, torch.float32)
    assert b.numel() >= 1000 and b.data_ptr() != ptr
    assert any(t.data_ptr() == ptr for t in ws._retired)  # still owned, so nothing else can be given its memory
    c = ws.get("counters", 16, torch.int32, zeroed=True)
    assert c.dtype == torch.int32 and int(c.abs().sum()) == 0

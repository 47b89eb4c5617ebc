"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice;
window groups give pages back; exhaustion is an error, not a crash."""
import random

import numpy as np
import pytest
import torch

from braidinfer_b200.cache import CacheError, CacheManager, GroupPages, PagePool, SlotTable, PAGE_SIZE
from braidinfer_b200.parts.spec import CacheRequest


def test_pool_hands_out_each_page_once_and_takes_it_back_once():
    p = PagePool(4)
    got = [p.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and p.available == 0 and p.in_use == 4
    with pytest.raises(CacheError, match="full"):
        p.alloc()
    p.free(got[1])
    with pytest.raises(CacheError, match="twice"):
        p.free(got[1])
    with pytest.raises(CacheError):
        p.free(99)
    assert p.alloc() == got[1]              # reused


def test_slots_are_reused_and_misuse_is_refused():
    t = SlotTable(2)
    a, b = t.alloc(), t.alloc()
    assert {a, b} == {0, 1} and t.available == 0
    with pytest.raises(CacheError, match="no free"):
        t.alloc()
    t.free(a)
    with pytest.raises(CacheError, match="twice"):
        t.free(a)
    assert t.alloc() == a and t.live_slots() == [0, 1]


def test_window_group_gives_back_blocks_the_window_has_passed():
    g = GroupPages(num_pages=8, page_size=4, kind="window", window=6)
    g.open(0)
    g.grow(0, 13)                     # a prompt of 13 tokens needs blocks 0..3 during its step
    assert g.pool.in_use == 4
    g.shrink(0, 13)                   # next query at 13 sees keys > 7: block 0 (0..3) and 1 (4..7) are dead
    assert g.blocks[0][:2] == [-1, -1] and g.blocks[0][2] >= 0 and g.pool.in_use == 2
    g.grow(0, 14); g.shrink(0, 14)    # keys > 8: nothing more
    assert g.pool.in_use == 2
    g.grow(0, 17); g.shrink(0, 17)    # block 4 added; keys > 11: block 2 (8..11) dead
    assert g.blocks[0] == [-1, -1, -1, g.blocks[0][3], g.blocks[0][4]] and g.pool.in_use == 2
    g.close(0)
    assert g.pool.in_use == 0
    full = GroupPages(8, 4, "full")
    full.open(3); full.grow(3, 13); full.shrink(3, 13)
    assert full.pool.in_use == 4


def plan(n_layers=2, window=None, state=0):
    req = CacheRequest("window" if window else "full", 2, 8, window)
    return [(req, None, state) for _ in range(n_layers)]


def test_manager_step_tables_and_lengths():
    m = CacheManager(plan(), max_tokens=PAGE_SIZE * 4, max_slots=3, dtype=torch.float32, device="cpu")
    a, b = m.alloc_slot(), m.alloc_slot()
    tables = m.begin_step([a, b], [70, 3])
    assert len(tables) == 1 and tables[0].shape == (2, 2)
    assert tables[0][0, 0] != tables[0][0, 1] and tables[0][1, 1] == -1
    m.end_step([a, b], [70, 3])
    assert m.length(a) == 70 and m.length(b) == 3 and m.pages_in_use() == [3]
    with pytest.raises(CacheError, match="full"):
        m.begin_step([b], [PAGE_SIZE * 2])          # would need 2 more pages, 1 is free
    assert m.pages_in_use() == [3]                   # a refused step reserves nothing
    with pytest.raises(CacheError, match="twice"):
        m.begin_step([a, a], [1, 1])
    m.free_slot(a)
    assert m.pages_in_use() == [1]
    with pytest.raises(CacheError):
        m.length(a)
    with pytest.raises(CacheError):
        m.free_slot(a)


def test_groups_by_request_and_shared_entries():
    full = CacheRequest("full", 2, 8, None)
    win = CacheRequest("window", 2, 8, 5)
    p = [(full, None, 0), (win, None, 16), (win, None, 0), (None, 0, 0), (full, None, 0)]
    m = CacheManager(p, max_tokens=128, max_slots=2, dtype=torch.float32, device="cpu")
    assert len(m.groups) == 2
    assert m.groups[0].storage.shape == (2, 2, 2, 2, PAGE_SIZE, 8)      # entries 0 and 4
    assert m.groups[1].storage.shape[0] == 2                            # entries 1 and 2
    v3, v0 = m.layer_view(3), m.layer_view(0)
    assert v3.read_only and not v0.read_only
    assert v3.storage.data_ptr() == v0.storage.data_ptr()               # entry 3 reads entry 0's cache
    assert m.state_view(1).shape == (2, 16) and m.state_view(0) is None
    s = m.alloc_slot()
    m.state_view(1)[s] = 7
    m.free_slot(s)
    s2 = m.alloc_slot()
    assert s2 == s and int(m.state_view(1)[s2].sum()) == 0              # state is zero when a slot is taken


def test_a_run_that_reads_another_runs_cache_must_fit_it():
    """Heads and head size must be the owner's, and the reader must not look further back than
    a windowed owner keeps pages for."""
    full, win5, win9 = CacheRequest("full", 2, 8, None), CacheRequest("window", 2, 8, 5), CacheRequest("window", 2, 8, 9)
    ok = [[(full, None, 0), (full, 0, 0)], [(full, None, 0), (win5, 0, 0)], [(win9, None, 0), (win5, 0, 0)],
          [(win5, None, 0), (win5, 0, 0)], [(win5, None, 0), (None, 0, 0)]]
    for plan in ok:
        CacheManager(plan, max_tokens=128, max_slots=2, dtype=torch.float32, device="cpu")
    bad = [([(win5, None, 0), (full, 0, 0)], "every earlier position"),
           ([(win5, None, 0), (win9, 0, 0)], "window of 9"),
           ([(full, None, 0), (CacheRequest("full", 4, 8, None), 0, 0)], "kv heads"),
           ([(full, None, 0), (CacheRequest("full", 2, 16, None), 0, 0)], "kv heads"),
           ([(None, None, 0), (full, 0, 0)], "keeps none")]
    for plan, word in bad:
        with pytest.raises(CacheError) as e:
            CacheManager(plan, max_tokens=128, max_slots=2, dtype=torch.float32, device="cpu")
        assert word in str(e.value), str(e.value)


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    m = CacheManager(plan(window=100), max_tokens=PAGE_SIZE * 12, max_slots=5, dtype=torch.float32, device="cpu")
    live = {}
    for _ in range(600):
        if live and rng.random() < 0.25:
            s = rng.choice(list(live))
            m.free_slot(s)
            del live[s]
        elif len(live) < 5 and rng.random() < 0.4:
            s = m.alloc_slot()
            assert s not in live
            live[s] = 0
        elif live:
            ss = rng.sample(list(live), rng.randint(1, len(live)))
            ns = [rng.randint(1, 90) for _ in ss]
            try:
                tables = m.begin_step(ss, ns)
            except CacheError:
                continue
            held = [p for row in tables[0] for p in row if p >= 0]
            assert len(held) == len(set(held))                           # no page held twice in a step
            m.end_step(ss, ns)
            for s, n in zip(ss, ns):
                live[s] += n
                assert m.length(s) == live[s]
        pages = [p for s in live for p in m.groups[0].pages.blocks[s] if p >= 0]
        assert len(pages) == len(set(pages)) == m.pages_in_use()[0]      # none lost, none shared
    for s in list(live):
        m.free_slot(s)
    assert m.pages_in_use() == [0] and m.slots.available == 5

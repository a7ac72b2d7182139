import random

import pytest
import torch

from nimbus_infer_rs_b200.cache import (PAGE, CacheError, PagePool, SequenceCache, SlotAllocator,
                                        pages_for)
from nimbus_infer_rs_b200.parts import KVRequest, StateRequest


def test_slots_none_lost_none_twice():
    a = SlotAllocator(5)
    got = [a.alloc() for _ in range(5)]
    assert sorted(got) == [0, 1, 2, 3, 4] and a.n_free == 0
    with pytest.raises(CacheError, match="no free sequence slot"):
        a.alloc()
    a.free(2)
    with pytest.raises(CacheError, match="not held"):
        a.free(2)                       # freed twice
    with pytest.raises(CacheError, match="not held"):
        a.free(17)                      # never handed out
    assert a.alloc() == 2               # used again
    rng = random.Random(0)
    held = set(got)
    for _ in range(2000):
        if held and (rng.random() < 0.5 or a.n_free == 0):
            s = rng.choice(sorted(held))
            a.free(s)
            held.remove(s)
        else:
            s = a.alloc()
            assert s not in held        # never held twice
            held.add(s)
        assert a.n_free + len(held) == 5 and a.held == frozenset(held)   # none lost


def test_page_pool():
    p = PagePool(4)
    x = p.alloc(3)
    assert len(set(x)) == 3
    with pytest.raises(CacheError, match="cache is full"):
        p.alloc(2)
    p.release(x[:1])
    with pytest.raises(CacheError, match="released twice"):
        p.release(x[:1])
    assert p.n_free == 2


def _cache(cache_tokens=512, max_seq_len=200, n_slots=None, state=True):
    kv = {0: KVRequest(2, 16), 1: KVRequest(2, 16), 2: KVRequest(1, 32, window=8)}
    st = {1: StateRequest(5)} if state else {}
    return SequenceCache(kv, st, cache_tokens=cache_tokens, max_seq_len=max_seq_len,
                         dtype=torch.float32, device="cpu", n_slots=n_slots)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.groups) == 2
    g0, g1 = c.groups
    assert g0.layers == [0, 1] and g1.layers == [2]
    assert g0.storage.shape == (2, 2, 8, 2, PAGE, 16) and g1.storage.shape == (1, 2, 8, 1, PAGE, 32)
    assert c.layer_kv(1).k.data_ptr() != c.layer_kv(0).k.data_ptr()
    assert c.layer_kv(2).window == 8 and c.layer_kv(3) is None
    assert c.layer_state(1).shape == (c.n_slots, 5) and c.layer_state(0) is None


def test_reserve_is_all_or_nothing_and_lengths_are_per_sequence():
    c = _cache(cache_tokens=4 * PAGE)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 65), (b, 10)])
    c.advance(a, 65)
    c.advance(b, 10)
    assert c.lens[a] == 65 and c.lens[b] == 10 and c.tokens_held() == 3 * PAGE
    free_before = [g.pool.n_free for g in c.groups]
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve([(a, 1), (b, 120)])         # b alone would need two more pages
    assert [g.pool.n_free for g in c.groups] == free_before      # nothing was taken
    with pytest.raises(CacheError, match="exceeds the longest sequence"):
        c.reserve([(a, 200)])
    with pytest.raises(CacheError, match="twice in one step"):
        c.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="not held"):
        c.reserve([(7, 1)])
    table = c.groups[0].block_table
    assert len(set(table[a, :2].tolist()) | set(table[b, :1].tolist())) == 3   # distinct pages


def test_slots_and_pages_come_back_and_state_is_cleared():
    c = _cache(cache_tokens=4 * PAGE, n_slots=2)
    a = c.alloc_slot()
    c.reserve([(a, 130)])
    c.advance(a, 130)
    c.layer_state(1)[a] = 7.0
    pages_a = c.groups[0].pages_of(a)
    b = c.alloc_slot()
    with pytest.raises(CacheError, match="no free sequence slot"):
        c.alloc_slot()
    c.free_slot(a)
    with pytest.raises(CacheError, match="not held"):
        c.free_slot(a)
    assert all(g.pool.n_free == 4 for g in c.groups)
    a2 = c.alloc_slot()
    assert a2 == a and c.lens[a2] == 0
    assert torch.all(c.layer_state(1)[a2] == 0)          # fixed-size state starts from zero
    c.reserve([(a2, 1), (b, 64)])
    assert set(c.groups[0].pages_of(a2)) <= set(pages_a)  # its old pages are used again
    assert pages_for(0) == 0 and pages_for(64) == 1 and pages_for(65) == 2


def test_random_traffic_never_loses_a_page():
    c = _cache(cache_tokens=16 * PAGE, max_seq_len=300, n_slots=6, state=False)
    rng = random.Random(1)
    live = {}
    for _ in range(500):
        if live and rng.random() < 0.3:
            s = rng.choice(sorted(live))
            c.free_slot(s)
            del live[s]
        elif len(live) < 6 and rng.random() < 0.5:
            live[c.alloc_slot()] = 0
        elif live:
            s = rng.choice(sorted(live))
            n = rng.randint(1, 70)
            try:
                c.reserve([(s, n)])
                c.advance(s, n)
                live[s] += n
            except CacheError:
                pass
        for g in c.groups:
            held = [p for s in live for p in g.pages_of(s)]
            assert len(held) == len(set(held))                       # no page held twice
            assert len(held) + g.pool.n_free == g.pool.n_pages       # none lost
            w = g.request.window
            for s, n in live.items():
                before_window = max(0, n - w + 1) // PAGE if w else 0
                assert len(g.pages_of(s)) == pages_for(n) - before_window


def test_a_window_group_gives_back_the_pages_before_its_window():
    kv = {0: KVRequest(2, 16), 1: KVRequest(2, 16, window=70)}
    c = SequenceCache(kv, {}, cache_tokens=8 * PAGE, max_seq_len=8 * PAGE, dtype=torch.float32,
                      device="cpu", n_slots=2)
    full, win = c.groups
    a = c.alloc_slot()
    c.reserve([(a, 200)])                      # a prompt needs all of its pages during its step
    assert len(full.pages_of(a)) == 4 and len(win.pages_of(a)) == 4
    first_pages = win.pages_of(a)
    c.advance(a, 200)
    # the token at position 200 reads keys 131..200: page 2 (128..191) and page 3
    assert len(full.pages_of(a)) == 4
    assert win.pages_of(a) == first_pages[2:] and win.pool.n_free == 6
    table = win.block_table[a].tolist()
    assert table[2:4] == first_pages[2:]       # the pages still in use stay where they were
    for step in range(200, 330):               # decode on: never more than three pages held
        c.reserve([(a, 1)])
        c.advance(a, 1)
        assert len(win.pages_of(a)) <= 3 and len(full.pages_of(a)) == pages_for(step + 1)
        first_key = max(0, c.lens[a] - 70 + 1)
        assert win._pages[a][first_key // PAGE] >= 0          # the window's first page is held
    b = c.alloc_slot()
    c.reserve([(b, 2 * PAGE)])                 # room that the window group gave back is used
    assert not set(win.pages_of(b)) & set(win.pages_of(a))
    c.free_slot(a)
    c.free_slot(b)
    assert win.pool.n_free == 8 and full.pool.n_free == 8

"""The cache's host-side bookkeeping: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from sonicboom_b200.cache import Cache, CacheError, CacheFull, FreeList, KVNeed, StateNeed


def make(max_tokens=640, window=0, n_slots=None, extra_group=False, state=False):
    needs = [KVNeed(2, 16, 0), KVNeed(2, 16, window), None]
    if extra_group:
        needs.append(KVNeed(1, 32, 0))
    states = [None] * len(needs)
    if state:
        states[2] = StateNeed((3,), torch.float32)
    return Cache(needs, states, max_tokens, torch.float32, "cpu", n_slots=n_slots)


def test_free_list_invariants():
    f = FreeList(4, "page")
    a = f.take(3)
    assert a == [0, 1, 2] and f.free_count == 1
    f.give_back([1])
    with pytest.raises(CacheError, match="freed twice"):
        f.give_back([1])
    with pytest.raises(CacheError, match="not of this pool"):
        f.give_back([9])
    with pytest.raises(CacheFull):
        f.take(3)
    assert f.take(2) == [1, 3]                 # a released id is used again first
    f.check()
    f._free.append(0)                          # corrupt it: 0 is held and now also free
    with pytest.raises(CacheError, match="both free and held"):
        f.check()


def test_groups_follow_needs():
    c = make(window=40, extra_group=True)
    assert len(c.groups) == 3
    assert c.group_of_entry == {0: 0, 1: 1, 3: 2}
    assert c.groups[0].storage.shape == (1, 10, 2, 2, 64, 16)
    assert c.groups[0].entry_storage(0).shape == (10, 2, 2, 64, 16)
    c2 = make(window=0)
    assert len(c2.groups) == 1 and c2.groups[0].entries == [0, 1]     # same need: one group


def test_pages_grow_with_length_and_come_back():
    c = make(max_tokens=640)
    s = c.open()
    c.reserve(s, 5); c.advance(s, 5)
    assert c.page_list(s, 0) == [0] and c.tokens_held() == 64
    c.reserve(s, 64); c.advance(s, 64)
    assert c.page_list(s, 0) == [0]
    c.reserve(s, 65); c.advance(s, 65)
    assert c.page_list(s, 0) == [0, 1] and c.tokens_held() == 128
    t = c.open()
    c.reserve(t, 200); c.advance(t, 200)
    assert c.page_list(t, 0) == [2, 3, 4, 5]
    c.check()
    c.close(s)
    assert c.groups[0].pool.free_count == 6
    u = c.open()
    assert u == s                              # the slot is used again
    c.reserve(u, 70)
    assert c.page_list(u, 0) == [0, 1]         # and so are its pages
    c.check()


def test_cannot_exceed_max_tokens_and_nothing_changes_on_failure():
    c = make(max_tokens=256)
    s, t = c.open(), c.open()
    c.reserve(s, 128); c.advance(s, 128)
    with pytest.raises(CacheFull):
        c.reserve(t, 129)
    assert c.page_list(t, 0) == [] and c.groups[0].pool.free_count == 2
    c.reserve(t, 128)
    c.check()
    with pytest.raises(CacheError, match="without pages"):
        c.advance(s, 500)
    with pytest.raises(CacheError, match="holds no sequence"):
        c.length(17)
    c.close(t)
    with pytest.raises(CacheError):
        c.close(t)                             # closed twice


def test_slots_run_out_and_return():
    c = make(max_tokens=640, n_slots=2)
    a, b = c.open(), c.open()
    with pytest.raises(CacheFull):
        c.open()
    c.close(a)
    assert c.open() == a
    c.check()


def test_window_group_gives_pages_back():
    c = make(max_tokens=64 * 20, window=40)
    s = c.open()
    c.reserve(s, 300); c.advance(s, 300)
    full, win = c.page_list(s, 0), c.page_list(s, 1)
    assert full == list(range(5))
    # the next query (position 300) sees keys 261..300; pages 0..3 hold keys up to 255
    assert win == [-1, -1, -1, -1, 4]
    assert c.groups[1].pool.free_count == 19
    for n in range(301, 400):
        c.reserve(s, n); c.advance(s, n)
        first_seen = n - 40 + 1                # lowest key the next query sees
        live = [i for i, p in enumerate(c.page_list(s, 1)) if p >= 0]
        assert live[0] == first_seen // 64 and live[-1] == (n - 1) // 64
    c.check()
    c.close(s)
    assert c.groups[1].pool.free_count == 20 and c.groups[0].pool.free_count == 20
    c.check()


def test_truncate_for_prefix_reuse():
    c = make(max_tokens=640, window=40)
    s = c.open()
    c.reserve(s, 100); c.advance(s, 100)
    assert c.truncate(s, 70) and c.length(s) == 70 and len(c.page_list(s, 0)) == 2
    c.reserve(s, 300); c.advance(s, 300)
    assert not c.truncate(s, 100)              # the window group no longer has those keys
    assert c.length(s) == 300
    c.check()


def test_state_rows_are_zeroed_on_reuse():
    c = make(state=True)
    assert set(c.state) == {2} and c.state[2].shape == (c.n_slots, 3)
    s = c.open()
    c.state[2][s] += 5
    c.close(s)
    assert c.open() == s and float(c.state[2][s].abs().sum()) == 0.0


def test_random_walk_keeps_invariants():
    rng = random.Random(3)
    c = make(max_tokens=64 * 12, window=70, n_slots=5, extra_group=True)
    live = {}
    for _ in range(600):
        op = rng.random()
        try:
            if op < 0.25:
                live[c.open()] = 0
            elif op < 0.8 and live:
                s = rng.choice(list(live))
                n = live[s] + rng.choice([1, 1, 1, 17, 64, 130])
                c.reserve(s, n); c.advance(s, n); live[s] = n
            elif live:
                s = rng.choice(list(live))
                c.close(s); del live[s]
        except CacheFull:
            pass
        c.check()
        assert {s: c.length(s) for s in live} == live
        assert c.tokens_held() <= 64 * 12
    for s in list(live):
        c.close(s)
    c.check()
    assert all(g.pool.free_count == g.pool.n for g in c.groups) and c.slots.free_count == 5

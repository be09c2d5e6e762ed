"""The cache's host side: no slot or page is lost, held twice or freed twice."""
import random

import pytest
import torch

from gpt_fast_b200.cache import Cache, CacheFull, CacheNeeds, FreeList, KVNeed, StateNeed


def make(max_tokens=64 * 10, **kw):
    needs = {0: CacheNeeds(kv=KVNeed(2, 16)), 1: CacheNeeds(kv=KVNeed(2, 16)),
             2: CacheNeeds(kv=KVNeed(1, 32, window=128)), 3: CacheNeeds(kv=KVNeed(2, 16), state=StateNeed((3, 4)))}
    return Cache(needs, torch.float32, "cpu", max_tokens=max_tokens, **kw)


def test_free_list_refuses_misuse():
    f = FreeList(3, "slot")
    a = f.alloc(2)
    assert sorted(a) == [0, 1] and f.n_free == 1
    with pytest.raises(CacheFull):
        f.alloc(2)
    assert f.n_free == 1                                   # a refused request takes nothing
    f.free([a[0]])
    with pytest.raises(ValueError, match="not in use"):
        f.free([a[0]])                                     # freed twice
    with pytest.raises(ValueError, match="not in use"):
        f.free([2])                                        # never allocated
    with pytest.raises(ValueError, match="not in use"):
        f.free([a[1], a[1]])                               # twice in one call
    assert f.in_use == {a[1]}


def test_groups_have_storage_of_their_own():
    c = make()
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    full = next(g for g in c.kv_groups if g.need.window is None)
    win = next(g for g in c.kv_groups if g.need.window == 128)
    assert full.entries == [0, 1, 3] and win.entries == [2]
    assert tuple(full.k_pool.shape) == (3, 10, 2, 64, 16) and tuple(win.k_pool.shape) == (1, 10, 1, 64, 32)
    assert c.view(1).kv.k_pool.data_ptr() == full.k_pool[1].data_ptr()
    assert c.view(3).state.shape == (c.n_slots, 3, 4) and c.view(0).state is None
    assert c.view(2).kv.page_table.data_ptr() != c.view(0).kv.page_table.data_ptr()


def test_slots_and_pages_come_back_and_are_used_again():
    c = make()
    s = c.begin(3)
    c.reserve(s[0], 65)          # 2 pages
    c.reserve(s[1], 1)           # 1 page
    c.reserve(s[2], 128)         # 2 pages
    assert c.pages_free == 5
    c.reserve(s[0], 100)         # still 2 pages
    assert c.pages_free == 5
    pages0 = list(c.kv_groups[0].slot_pages[s[0]])
    c.end([s[0]])
    assert c.pages_free == 7 and c.slots.n_free == c.n_slots - 2
    assert (c.kv_groups[0].table_host[s[0]] == -1).all()
    t = c.begin(1)
    c.reserve(t[0], 64 * 2)
    assert t[0] == s[0] and sorted(c.kv_groups[0].slot_pages[t[0]]) == sorted(pages0)      # reused
    with pytest.raises(ValueError):
        c.end([s[0], s[0]])
    c.end([s[1], s[2], t[0]])
    assert c.pages_free == c.n_pages and c.slots.n_free == c.n_slots
    with pytest.raises(ValueError):
        c.end([s[1]])


def test_limits_are_errors_before_anything_changes():
    c = make(max_tokens=64 * 4, max_seqs=2, max_seq_len=128)
    assert (c.n_pages, c.n_slots, c.max_pages) == (4, 2, 2)
    s = c.begin(2)
    with pytest.raises(CacheFull):
        c.begin(1)
    with pytest.raises(CacheFull, match="longest sequence"):
        c.reserve(s[0], 129)
    c.reserve(s[0], 128)
    c.reserve(s[1], 128)
    assert c.pages_free == 0 and not c.can_reserve([1])
    with pytest.raises(ValueError, match="not in use"):
        c.reserve(5, 1)
    c.end(s)
    assert c.can_reserve([128, 128]) and not c.can_reserve([128, 128, 1]) and not c.can_reserve([129])


def test_state_is_zero_when_a_slot_is_handed_out():
    c = make()
    s = c.begin(2)
    c.view(3).state[s[0]] = 7.0
    c.lengths[s[0]] = 33
    c.end(s)
    again = c.begin(2)
    assert set(again) == set(s)
    assert float(c.view(3).state[s[0]].abs().sum()) == 0.0 and int(c.lengths[s[0]]) == 0


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make(max_tokens=64 * 40, max_seqs=12)
    live = {}
    for _ in range(600):
        if live and rng.random() < 0.4:
            s = rng.choice(list(live))
            c.end([s])
            del live[s]
        elif rng.random() < 0.5 and c.slots.n_free:
            want = rng.randint(1, 400)
            if c.can_reserve([want]):
                s = c.begin(1)[0]
                assert s not in live
                c.reserve(s, want)
                live[s] = want
        elif live:
            s = rng.choice(list(live))
            more = live[s] + rng.randint(1, 100)
            try:
                c.reserve(s, more)
                live[s] = more
            except CacheFull:
                pass
        for g in c.kv_groups:
            held = [p for s in live for p in g.slot_pages.get(s, [])]
            assert len(held) == len(set(held))                                  # no page held twice
            assert len(held) + g.pages.n_free == c.n_pages                      # none lost
            for s, n in live.items():
                assert len(g.slot_pages[s]) == -(-n // 64)
        assert len(live) + c.slots.n_free == c.n_slots
    c.end(list(live))
    assert c.pages_free == c.n_pages

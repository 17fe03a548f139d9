"""The cache's bookkeeping on the host: no slot lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from yalm_b200.cache import Cache, CacheNeed, SlotAllocator, SlotError


def test_slots_are_handed_out_once_and_come_back():
    a = SlotAllocator(4)
    s = a.acquire(3)
    assert sorted(s) == [0, 1, 2] and a.free_count == 1
    with pytest.raises(SlotError, match="only 1 of 4"):
        a.acquire(2)
    a.release([s[1]])
    assert a.free_count == 2 and a.held == [0, 2]
    again = a.acquire(2)
    assert sorted(again) == [1, 3]
    a.check()


def test_double_free_and_foreign_slots_raise():
    a = SlotAllocator(3)
    s = a.acquire(2)
    a.release([s[0]])
    with pytest.raises(SlotError, match="not held"):
        a.release([s[0]])
    with pytest.raises(SlotError, match="does not exist"):
        a.release([7])
    with pytest.raises(SlotError, match="twice"):
        a.release([s[1], s[1]])
    assert a.held == [s[1]]                      # the failed call released nothing
    with pytest.raises(SlotError):
        SlotAllocator(0)


def test_random_traffic_never_loses_or_duplicates_a_slot():
    rng = random.Random(0)
    a = SlotAllocator(9)
    mine = []
    for _ in range(2000):
        if mine and (rng.random() < 0.5 or a.free_count == 0):
            k = rng.randint(1, len(mine))
            out = [mine.pop(rng.randrange(len(mine))) for _ in range(k)]
            a.release(out)
        else:
            got = a.acquire(rng.randint(1, a.free_count))
            assert not set(got) & set(mine)
            mine.extend(got)
        a.check()
        assert sorted(mine) == a.held and a.free_count == 9 - len(mine)


def test_groups_have_storage_of_their_own_and_state_is_zeroed():
    needs = {0: CacheNeed("kv", kv_heads=2, head_dim=16),
             1: CacheNeed("kv", kv_heads=2, head_dim=16, window=8),
             2: CacheNeed("kv", kv_heads=2, head_dim=16),
             3: CacheNeed("state", state_shape=(4, 3))}
    c = Cache(needs, n_slots=3, context=32, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 3
    full, ring, state = c.view(0), c.view(1), c.view(3)
    # no bound on the tokens held: one block per sequence, [slots, kv heads, capacity, head size]
    assert full.k.shape == (3, 2, 32, 16) and ring.k.shape == (3, 2, 8, 16)
    assert full.capacity == 32 and ring.capacity == 8 and full.pages is None
    # a bound below slots x capacity: pages of 64 positions, [kv heads, pages, 64, head size]
    p = Cache({0: CacheNeed("kv", kv_heads=2, head_dim=16)}, 3, 256, torch.float32, "cpu", max_tokens=320)
    assert p.view(0).k.shape == (2, 5, 64, 16) and p.view(0).pages.shape == (3, 4)
    assert p.bytes() == Cache.bytes_needed({0: CacheNeed("kv", kv_heads=2, head_dim=16)}, 3, 256,
                                           torch.float32, 320)
    assert c.view(2).k.data_ptr() != full.k.data_ptr()          # same group, own layer plane
    assert state.state.shape == (3, 4, 3)
    assert c.bytes() == Cache.bytes_needed(needs, 3, 32, torch.float32)
    s = c.acquire(2)
    state.state[s[0]] += 5.0
    c.slot_pos[s[0]] = 17
    c.host_pos[s[0]] = 17
    c.release(s)
    t = c.acquire(3)                                            # slots come back, reset
    assert sorted(t) == [0, 1, 2]
    assert c.slot_pos.tolist() == [0, 0, 0] and c.host_pos == [0, 0, 0]
    assert float(c.view(3).state.abs().sum()) == 0.0
    with pytest.raises(SlotError):
        c.acquire(1)
    with pytest.raises(KeyError):
        Cache({0: needs[0]}, 1, 8, torch.float32, "cpu").view(5)


def test_pages_follow_the_tokens_and_come_back():
    """A sequence takes a page when it grows into it; a windowed group never takes more
    than its ring needs; release returns every page; a request beyond the pool changes
    nothing and says so."""
    from yalm_b200.cache import CacheFull, PAGE
    needs = {0: CacheNeed("kv", kv_heads=1, head_dim=8),
             1: CacheNeed("kv", kv_heads=1, head_dim=8, window=100)}
    c = Cache(needs, n_slots=4, context=1000, dtype=torch.float32, device="cpu", max_tokens=640)
    assert c.free_pages() == [10]                 # 640 tokens; the four rings of 100 rows fit whole
    assert c.view(1).pages is None and c.view(1).k.shape == (4, 1, 100, 8)
    a, b = c.acquire(2)
    c.ensure([a, b], [1, 130])
    assert c.free_pages() == [10 - 1 - 3]
    c.ensure([a, b], [64, 192])                   # still inside the pages they hold
    assert c.free_pages() == [6]
    c.ensure([a], [65])
    assert c.free_pages() == [5]
    c.sync_tables()
    full = c.view(0)
    held = c.groups[0]["held"]
    assert full.pages[a, :2].tolist() == held[a] and full.pages[b, :3].tolist() == held[b]
    assert len(set(held[a]) | set(held[b])) == 5  # no page held twice
    with pytest.raises(CacheFull, match="more pages"):
        c.ensure([a, b], [200, 450])              # 2 + 5 more of the first group: only 5 are free
    assert c.free_pages() == [5]                  # nothing was taken
    c.release([a])
    assert c.free_pages() == [7]
    (d,) = c.acquire(1)
    c.ensure([d], [PAGE * 7])
    assert c.free_pages() == [0]
    c.release([b, d])
    assert c.free_pages() == [10]
    c.groups[0]["pool"].check()


def test_random_page_traffic_never_loses_or_duplicates_a_page():
    rng = random.Random(1)
    needs = {0: CacheNeed("kv", kv_heads=1, head_dim=8)}
    c = Cache(needs, n_slots=5, context=640, dtype=torch.float32, device="cpu", max_tokens=1600)
    from yalm_b200.cache import CacheFull
    live = {}
    for _ in range(600):
        if live and rng.random() < 0.3:
            s = rng.choice(sorted(live))
            c.release([s])
            del live[s]
        elif len(live) < 5 and rng.random() < 0.4:
            (s,) = c.acquire(1)
            live[s] = 0
        elif live:
            s = rng.choice(sorted(live))
            n = min(640, live[s] + rng.randint(1, 200))
            try:
                c.ensure([s], [n])
                live[s] = n
            except CacheFull:
                pass
        held = [p for s in live for p in c.groups[0]["held"][s]]
        assert len(held) == len(set(held)) == 25 - c.free_pages()[0]
        assert all(len(c.groups[0]["held"][s]) == -(-live[s] // 64) for s in live)
        c.groups[0]["pool"].check()

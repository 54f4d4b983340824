"""The cache's bookkeeping: no page or slot lost, held twice or freed twice (CPU)."""
import random

import pytest
import torch

from synaptix_b200.cache import (PAGE_TOKENS, Cache, CacheFull, KVRequest, PagePool, SequenceSlots,
                                 SlotError, StateRequest, pages_for)


def test_pool_hands_out_each_page_once():
    p = PagePool(5)
    a = p.alloc(3)
    b = p.alloc(2)
    assert sorted(a + b) == [0, 1, 2, 3, 4] and p.n_free == 0
    with pytest.raises(CacheFull):
        p.alloc(1)
    p.free(a)
    assert p.n_free == 3
    with pytest.raises(SlotError, match="twice"):
        p.free([a[0]])
    with pytest.raises(SlotError):
        p.free([99])
    with pytest.raises(SlotError, match="twice"):
        p.free([b[0], b[0]])
    assert p.n_free == 3 and sorted(p.held()) == sorted(b)
    # a failed alloc takes nothing
    with pytest.raises(CacheFull):
        p.alloc(4)
    assert p.n_free == 3


def test_freed_pages_are_reused_first():
    p = PagePool(8)
    a = p.alloc(2)
    p.free(a)
    assert set(p.alloc(2)) == set(a)


def check_invariants(slots: SequenceSlots):
    for g, pool in enumerate(slots.pools):
        held = []
        for s in slots.live():
            held += [p for p in slots.table(s, g) if p >= 0]
        assert len(held) == len(set(held)), "a page is held twice"
        assert sorted(held) == sorted(pool.held()), "a page is lost or held by nobody"
        assert len(held) + pool.n_free == pool.n_pages
    assert slots.n_live + len(slots._free_slots) == slots.max_seqs


def test_slots_random_walk_keeps_every_page_accounted():
    rng = random.Random(0)
    slots = SequenceSlots(6, [PagePool(40), PagePool(40)], [None, 100])
    live = []
    for _ in range(3000):
        op = rng.random()
        if op < 0.15 and slots.n_live < 6:
            live.append(slots.open())
        elif op < 0.25 and live:
            s = live.pop(rng.randrange(len(live)))
            slots.close(s)
            with pytest.raises(SlotError):
                slots.close(s)
            with pytest.raises(SlotError):
                slots.length(s)
        elif live:
            s = rng.choice(live)
            n = rng.choice([1, 1, 1, 5, 64, 130])
            before = (slots.length(s), [list(slots.table(s, g)) for g in range(2)], [p.n_free for p in slots.pools])
            try:
                slots.reserve(s, n)
            except CacheFull:
                after = (slots.length(s), [list(slots.table(s, g)) for g in range(2)], [p.n_free for p in slots.pools])
                assert before == after, "a failed reserve changed something"
                continue
            slots.advance(s, n)
            assert len(slots.table(s, 0)) == pages_for(slots.length(s))
        check_invariants(slots)
    for s in live:
        slots.close(s)
    check_invariants(slots)
    assert all(p.n_free == p.n_pages for p in slots.pools)


def test_slot_table_full_and_slot_reuse():
    slots = SequenceSlots(2, [PagePool(4)])
    a, b = slots.open(), slots.open()
    with pytest.raises(CacheFull, match="slots"):
        slots.open()
    slots.close(a)
    assert slots.open() == a          # the slot that was given back is used again
    with pytest.raises(SlotError):
        slots.advance(b, 1)           # no page reserved


def test_reserve_many_is_all_or_nothing():
    slots = SequenceSlots(3, [PagePool(3)])
    a, b = slots.open(), slots.open()
    with pytest.raises(CacheFull):
        slots.reserve_many([a, b], [65, 129])     # 2 + 3 pages wanted, 3 there
    assert slots.pools[0].n_free == 3 and slots.table(a, 0) == [] and slots.table(b, 0) == []
    slots.reserve_many([a, b], [65, 64])
    assert slots.pools[0].n_free == 0


def test_windowed_group_gives_pages_back_while_running():
    W = 100
    slots = SequenceSlots(1, [PagePool(64), PagePool(64)], [None, W])
    s = slots.open()
    for _ in range(1000):
        slots.reserve(s, 1)
        slots.advance(s, 1)
        n = slots.length(s)
        full, win = slots.table(s, 0), slots.table(s, 1)
        assert all(p >= 0 for p in full)
        # every key a later query can see is still held: keys > n - W (query at position >= n)
        first_needed = max(0, n - W + 1)
        for i, p in enumerate(win):
            if i * PAGE_TOKENS + PAGE_TOKENS - 1 >= first_needed:
                assert p >= 0, f"page {i} was released while key {first_needed} is still visible"
        held = sum(p >= 0 for p in win)
        assert held <= pages_for(W) + 2
    slots.close(s)
    assert slots.pools[1].n_free == 64 and slots.pools[0].n_free == 64


def test_cache_groups_requests_and_resets_state():
    reqs = [KVRequest(2, 16), KVRequest(2, 16, window=8), KVRequest(2, 16), StateRequest((3, 4)), None]
    c = Cache(reqs, max_tokens=200, max_seqs=3, dtype=torch.float32, device="cpu")
    assert c.n_pages == 5 and c.max_tokens == 256      # 4 pages to hand out + the never-used page 0
    assert len(c.kv_groups) == 2 and c.n_block_tables == 2
    assert c.kv_bytes_per_token == 3 * 2 * 2 * 16 * 4               # three layers of keys and values, 2 heads of 16 floats
    v0, v1, v2 = c.view(0), c.view(1), c.view(2)
    assert v0.group == v2.group == 0 and v1.group == 1 and v1.window == 8
    assert v0.k.shape == (5, 2, PAGE_TOKENS, 16)
    assert all(0 not in c.slots.pools[g].alloc(4) for g in range(2))
    assert v0.k.data_ptr() != v2.k.data_ptr() and v0.k.data_ptr() != v1.k.data_ptr()
    assert c.view(4) is None
    st = c.view(3)
    # a row per slot and one more that no sequence owns (rows that pad a captured step carry that slot number)
    assert st.shape == (4, 3, 4) and c.spare_slot == 3
    assert c.spare_slot not in [c.slots.open() for _ in range(3)]
    for x in (0, 1, 2):
        c.slots.close(x)
    s = c.open()
    st[s] += 5.0
    c.close(s)
    s2 = c.open()
    assert s2 == s and float(c.view(3)[s2].abs().sum()) == 0.0     # a reused slot starts from zero state


def test_cache_without_keys_still_counts_lengths():
    c = Cache([StateRequest((2,))], max_tokens=128, max_seqs=2, dtype=torch.float32, device="cpu")
    s = c.open()
    c.slots.reserve(s, 70)
    c.slots.advance(s, 70)
    assert c.slots.length(s) == 70

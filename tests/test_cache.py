"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; groups; windows."""
import random

import pytest
import torch

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.cache import PAGE, Cache, CacheError, CacheFull, PagePool, SlotTable, pages_for
from bitnet_c_b200.parts import KvRequest, StateRequest


def make(kv, cache_of=None, states=None, max_tokens=640, max_positions=512, max_seqs=4):
    n = len(kv)
    return Cache(kv, cache_of or [None] * n, states or [None] * n, max_tokens, max_positions, torch.bfloat16,
                 None, max_seqs=max_seqs, allocate=False)


def test_page_pool_never_loses_or_doubles():
    p = PagePool(10)
    a = p.alloc(4)
    b = p.alloc(6)
    assert sorted(a + b) == list(range(10)) and p.n_free == 0
    with pytest.raises(CacheFull):
        p.alloc(1)
    p.free(a)
    with pytest.raises(CacheError, match="freed twice"):
        p.free([a[0]])
    with pytest.raises(CacheError, match="does not exist"):
        p.free([99])
    p.check()
    assert sorted(p.alloc(4)) == sorted(a)


def test_slot_table():
    s = SlotTable(3)
    a, b, c = s.open(), s.open(), s.open()
    assert {a, b, c} == {0, 1, 2}
    with pytest.raises(CacheFull):
        s.open()
    s.close(b)
    with pytest.raises(CacheError, match="not open"):
        s.close(b)
    with pytest.raises(CacheError):
        s.length(b)
    assert s.open() == b  # given back and used again
    s.check()


def test_reserve_advance_close_cycle_many_times():
    req = KvRequest(2, 16)
    c = make([req, req, req])
    assert len(c.groups) == 1 and c.groups[0].entries == [0, 1, 2]
    rng = random.Random(0)
    live = {}
    for _ in range(500):
        if live and (rng.random() < 0.3 or c.slots.n_free == 0):
            slot = rng.choice(list(live))
            c.close(slot)
            del live[slot]
        elif rng.random() < 0.5 or not live:
            live[c.open()] = 0
        else:
            slot = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 100])
            try:
                c.reserve(slot, n)
                c.advance(slot, n)
                live[slot] += n
            except CacheFull:
                pass
        c.check()
        for slot, n in live.items():
            assert c.length(slot) == n
            assert len(c.groups[0].held.get(slot, {})) == pages_for(n)
    for slot in list(live):
        c.close(slot)
    c.check()
    assert c.groups[0].pool.n_free == c.groups[0].pool.n_pages and c.slots.n_free == 4


def test_failed_reserve_changes_nothing():
    c = make([KvRequest(1, 16)], max_tokens=128, max_positions=4096)
    a, b = c.open(), c.open()
    c.reserve(a, 64)
    c.advance(a, 64)
    c.reserve(b, 10)
    c.advance(b, 10)
    with pytest.raises(CacheFull):
        c.reserve(a, 1)  # would need a third page
    assert c.length(a) == 64 and len(c.groups[0].held[a]) == 1
    c.check()
    small = make([KvRequest(1, 16)], max_positions=100)
    with pytest.raises(CacheFull, match="exceed the context"):
        small.reserve(small.open(), 101)
    small.check()


def test_groups_have_storage_of_their_own_and_readers_share_a_plane():
    full, win = KvRequest(2, 16), KvRequest(2, 16, window=70)
    c = make([full, win, None, full, win], cache_of=[None, None, None, 0, None],
             states=[None, None, StateRequest((3, 5)), None, None])
    assert [g.request for g in c.groups] == [full, win]
    assert c.groups[0].entries == [0] and c.groups[1].entries == [1, 4]
    assert c._reader == {3: 0}
    slot = c.open()
    for _ in range(5):
        c.reserve(slot, 64)
        c.advance(slot, 64)
        c.check()
    # 320 tokens: the full group holds 5 pages; the window group only pages that still hold one
    # of the last 70 keys (positions 251..319 -> pages 3 and 4)
    assert sorted(c.groups[0].held[slot]) == [0, 1, 2, 3, 4]
    assert sorted(c.groups[1].held[slot]) == [3, 4]
    c.close(slot)
    c.check()
    with pytest.raises(CacheError, match="which has none"):
        make([None, full], cache_of=[None, 0])
    with pytest.raises(CacheError, match="cannot read"):
        make([full, KvRequest(4, 16)], cache_of=[None, 0])


def test_sizes_round_up_to_pages():
    c = make([KvRequest(1, 16)], max_tokens=100)
    assert c.max_tokens == 128 and c.groups[0].pool.n_pages == 2 and PAGE == 64
    assert c.tokens_free() == 128

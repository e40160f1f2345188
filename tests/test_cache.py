"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice; groups with
different needs have storage of their own; rings; capacity errors; fixed-size state."""
from __future__ import annotations

import random

import pytest
import torch

from janis_b200.cache.cache import (PAGE, CacheError, CacheFull, KVNeed, ModelCache, PagePool, StateNeed)


def gemma_like(n_layers=4, window=100):
    return [{"kv": KVNeed(2, 16, window if i % 2 == 0 else None)} for i in range(n_layers)]


def make(max_tokens=10 * PAGE, **kw):
    return ModelCache(gemma_like(), max_tokens, kw.pop("max_ctx", 4096), torch.float32, "cpu", **kw)


def test_page_pool_never_hands_out_twice_or_takes_back_twice():
    p = PagePool(5)
    a = p.alloc(3)
    b = p.alloc(2)
    assert sorted(a + b) == [0, 1, 2, 3, 4] and p.n_free == 0
    with pytest.raises(CacheFull):
        p.alloc(1)
    p.free(a)
    with pytest.raises(CacheError, match="freed but not held"):
        p.free([a[0]])
    with pytest.raises(CacheError, match="freed but not held"):
        p.free([99])
    p.audit(b)
    with pytest.raises(CacheError):
        p.audit(b + b[:1])


def test_groups_by_need_have_their_own_storage():
    c = make()
    assert len(c.kv_groups) == 2
    full = c.kv_groups[KVNeed(2, 16, None)]
    ring = c.kv_groups[KVNeed(2, 16, 100)]
    assert full.lines == [1, 3] and ring.lines == [0, 2]
    assert full.ring_len == 0 and ring.ring_len == 2 * PAGE          # a window of 100 lives in a ring of 128
    assert full.k.shape == (2, 10, 2, PAGE, 16) and ring.pages_per_seq == 2
    assert full.k.data_ptr() != ring.k.data_ptr()
    l0, l1 = c.line(0), c.line(1)
    assert l0["kv"].ring_len == 128 and l0["kv"].window == 100 and l1["kv"].ring_len == 0
    assert l0["kv"].k.shape == (ring.k.shape[1], 2, PAGE, 16)


def test_slots_are_given_back_and_used_again():
    c = make(max_seqs=3)
    s = [c.alloc_slot() for _ in range(3)]
    assert sorted(s) == [0, 1, 2]
    with pytest.raises(CacheFull, match="no free slot"):
        c.alloc_slot()
    c.free_slot(s[1])
    with pytest.raises(CacheError, match="freed but not in use"):
        c.free_slot(s[1])
    assert c.alloc_slot() == s[1]
    with pytest.raises(CacheError, match="not in use"):
        c.reserve(77, 5)
    c.audit()


def test_pages_follow_each_sequences_own_length():
    c = make()
    full = c.kv_groups[KVNeed(2, 16, None)]
    ring = c.kv_groups[KVNeed(2, 16, 100)]
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve(a, 1)
    c.reserve(b, 3 * PAGE + 1)
    assert len(full.held[a]) == 1 and len(full.held[b]) == 4
    assert len(ring.held[a]) == 1 and len(ring.held[b]) == 2           # the ring never grows past its pages
    c.advance(a, 1)
    c.advance(b, 3 * PAGE + 1)
    c.reserve(a, PAGE)                                                  # still the first page
    assert len(full.held[a]) == 1
    c.reserve(a, PAGE + 1)
    assert len(full.held[a]) == 2
    assert set(full.held[a]).isdisjoint(full.held[b])
    assert full.table_host[a, :2].tolist() == full.held[a]
    with pytest.raises(CacheFull, match="cache is full"):
        c.reserve(a, 7 * PAGE)                                          # 4 + 7 > 10 pages
    c.audit()
    c.free_slot(b)
    c.reserve(a, 7 * PAGE)
    c.audit()
    with pytest.raises(CacheError, match="cannot shrink"):
        c.advance(a, 0)


def test_context_limit_and_room():
    c = make(max_ctx=200)
    s = c.alloc_slot()
    with pytest.raises(CacheFull, match="context holds 200"):
        c.reserve(s, 201)
    assert c.can_hold([200, 64]) and not c.can_hold([201])
    assert not c.can_hold([PAGE] * 11)                                  # 11 pages of 10


def test_state_groups_are_zeroed_when_a_slot_is_handed_out():
    needs = [{"state": StateNeed((3, 2))}, {"kv": KVNeed(1, 16, None), "state": StateNeed((3, 2))},
             {"other": StateNeed((5,), torch.int32)}]
    c = ModelCache(needs, 4 * PAGE, 1024, torch.float32, "cpu", max_seqs=2)
    assert len(c.state_groups) == 2 and len(c.kv_groups) == 1
    s = c.alloc_slot()
    line = c.line(1)
    line["state"].data[s] += 5.0
    assert c.state_groups[StateNeed((3, 2))].data[1, s].sum() == 30.0
    assert c.line(0)["state"].data[s].sum() == 0                        # another line of the same group
    c.free_slot(s)
    t = c.alloc_slot()
    assert t == s and c.line(1)["state"].data[t].sum() == 0
    assert c.line(2)["other"].data.dtype == torch.int32


def test_random_traffic_loses_nothing():
    rnd = random.Random(3)
    c = make(max_tokens=40 * PAGE, max_seqs=12)
    live = {}
    for _ in range(3000):
        r = rnd.random()
        if r < 0.25 and c.n_free_slots:
            live[c.alloc_slot()] = 0
        elif r < 0.45 and live:
            s = rnd.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rnd.choice(list(live))
            n = live[s] + rnd.choice([1, 1, 1, 30, 200])
            try:
                c.reserve(s, n)
                c.advance(s, n)
                live[s] = n
            except CacheFull:
                pass
        c.audit()
        assert sorted(live) == c.live_slots()
    for s in list(live):
        c.free_slot(s)
    c.audit()
    for g in c.kv_groups.values():
        assert g.pool.n_free == g.pool.n_pages and not g.held


def test_the_planned_size_is_what_the_groups_hold():
    needs = [{"kv": KVNeed(2, 16, 8)}, {"kv": KVNeed(2, 16)}, {"kv": KVNeed(2, 16, 8), "s": StateNeed((5,), torch.float32)}]
    c = ModelCache(needs, 10 * 64, 512, torch.bfloat16, "cpu", max_seqs=3)
    assert c.planned_bytes == c.bytes()
    # windowed lines hold a ring per sequence (here one page each), the others every page
    assert c.bytes() == 2 * 2 * 3 * 2 * 64 * 16 * 2 + 2 * 1 * 10 * 2 * 64 * 16 * 2 + 3 * 5 * 4


@pytest.mark.gpu
def test_a_cache_the_device_has_no_room_for_is_refused_with_its_sizes():
    """Asked for more tokens than the device can hold, the cache says what it would need and what is free,
    before it allocates anything (no out-of-memory error from the allocator, nothing left half built)."""
    needs = [{"kv": KVNeed(16, 256, 4096)}, {"kv": KVNeed(16, 256)}] * 20
    before = torch.cuda.memory_allocated()
    with pytest.raises(CacheFull, match=r"needs \d+\.\d+ GiB .* the device has \d+\.\d+ GiB free"):
        ModelCache(needs, 40_000_000, 8192, torch.bfloat16, "cuda:0", max_seqs=64)
    assert torch.cuda.memory_allocated() == before
    small = ModelCache(needs, 128, 8192, torch.bfloat16, "cuda:0", max_seqs=2)
    assert small.bytes() == small.planned_bytes

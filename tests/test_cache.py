"""The cache manager without tensors: no page lost, held twice or freed twice, under random orders."""

from __future__ import annotations

import random

import pytest
from hypothesis import given, settings, strategies as st

from edgerag_b200.cache.allocator import AllocatorError, DoubleFreeError, OutOfPagesError, UnitAllocator
from edgerag_b200.cache.manager import NO_PAGE, CacheLayout, CacheManager, KVGroupSpec, StateSpec


def layout(window: int = 0, two_groups: bool = False) -> CacheLayout:
    groups = [KVGroupSpec(2, 2, 16, 0)]
    placement = [(0, 0), (0, 1)]
    if two_groups:
        groups.append(KVGroupSpec(1, 1, 32, window))
        placement.append((1, 0))
    elif window:
        groups = [KVGroupSpec(2, 2, 16, window)]
    return CacheLayout(groups=groups, placement=placement, states=[StateSpec("s@0", (4,))])


def test_allocator_basics():
    a = UnitAllocator(4)
    assert a.allocate(2) == [0, 1] and a.num_free == 2
    with pytest.raises(OutOfPagesError):
        a.allocate(3)
    assert a.num_free == 2 and a.stats.failed_allocations == 1     # all or nothing
    a.free([1])
    assert a.allocate(1) == [1]                                     # LIFO: just freed, next out
    with pytest.raises(DoubleFreeError):
        a.free([2])
    with pytest.raises(DoubleFreeError):
        a.free([0, 0])
    assert a.is_held(0)                                             # a failed free changes nothing
    with pytest.raises(AllocatorError):
        a.free([9])
    a.free([0, 1])
    a.check_invariants()
    assert a.num_free == 4 and a.stats.peak_used == 2


@settings(max_examples=200, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["alloc", "free"]), st.integers(0, 6)), max_size=60), st.integers(1, 12))
def test_allocator_random_sequences(ops, capacity):
    a = UnitAllocator(capacity)
    held: list[int] = []
    for op, n in ops:
        if op == "alloc":
            try:
                got = a.allocate(n)
                assert len(got) == n and not set(got) & set(held)
                held += got
            except OutOfPagesError:
                assert n > capacity - len(held)
        else:
            give, held = held[:n], held[n:]
            a.free(give)
        a.check_invariants()
        assert a.num_used == len(held)
    a.free(held)
    assert a.num_free == capacity


def test_growth_then_advance_and_slots():
    m = CacheManager(layout(), page_size=8, num_pages=10, max_requests=2)
    rc = m.admit("x")
    assert m.pages_to_grow("x", 17) == [3]
    m.grow("x", 17)
    assert [r.tolist() for r in m.slots_for("x", 3)] == [[rc.tables[0].pages[0] * 8 + i for i in range(3)]]
    m.advance("x", 17)
    assert rc.num_tokens == 17 and m.pages_to_grow("x", 7) == [0] and m.pages_to_grow("x", 8) == [1]
    assert [r.tolist() for r in m.slots_for("x", 1)] == [[rc.tables[0].pages[2] * 8 + 1]]
    with pytest.raises(AllocatorError):
        m.advance("x", 9)                      # advancing past the pages: grow first
    m.admit("y")
    with pytest.raises(OutOfPagesError):
        m.grow("y", 8 * 8)                     # 8 pages wanted, 7 free
    assert m.held_pages("y") == [0]            # a failed growth leaves nothing behind
    with pytest.raises(OutOfPagesError):
        m.admit("z")                           # both state slots are taken
    with pytest.raises(AllocatorError):
        m.admit("x")
    m.release("x")
    m.check_invariants()
    assert m.free_pages() == [10] and sorted(m.drain_new_slots()) == [0, 1]
    m.grow("y", 8 * 8)
    assert m.requests["y"].tables[0].pages[:3] == [2, 1, 0]       # pages just given back come first


def test_window_gives_pages_back_early():
    m = CacheManager(layout(window=10), page_size=4, num_pages=8, max_requests=1)
    rc = m.admit("w")
    total = 0
    for n in (6, 1, 1, 9, 1, 1, 1, 14):
        m.grow("w", n)
        assert all(p != NO_PAGE for p in rc.tables[0].pages[(total // 4):])   # pages to be written are live
        m.advance("w", n)
        total += n
        m.check_invariants()
        # keys <= total - window are dead; a page goes back once its last key is dead
        dead_pages = max(0, (total - 10 + 1) // 4)
        assert rc.tables[0].first_live == dead_pages
        assert rc.tables[0].pages[:dead_pages] == [NO_PAGE] * dead_pages
        assert m.held_pages("w") == [m.pages_for(total) - dead_pages]
    assert m.peak_pages(1000, 14) == [min(250, m.pages_for(24) + 1)]
    m.release("w")
    assert m.free_pages() == [8] and len(m.drain_freed()) == 9   # every page came back exactly once


def test_groups_have_pages_of_their_own():
    m = CacheManager(layout(window=8, two_groups=True), page_size=4, num_pages=[6, 3], max_requests=2)
    m.admit("a")
    m.grow("a", 12)
    m.advance("a", 12)
    assert m.held_pages("a") == [3, 2]          # the windowed group already gave page 0 back
    assert m.free_pages() == [3, 1]
    m.admit("b")
    assert not m.can_grow("b", 8)               # group 1 has one page left, two are needed
    with pytest.raises(OutOfPagesError):
        m.grow("b", 8)
    assert m.held_pages("b") == [0, 0]          # nothing taken in group 0 either
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    """Admit, grow, advance and release in random orders; invariants hold after every operation."""
    rng = random.Random(seed)
    windowed = seed % 2 == 1
    m = CacheManager(layout(window=12 if windowed else 0, two_groups=True), page_size=4,
                     num_pages=[40, 25], max_requests=5)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 5:
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            if m.can_grow(rid, n):
                m.grow(rid, n)
                assert len(m.slots_for(rid, n)[0]) == n
                m.advance(rid, n)
                live[rid] += n
            else:
                with pytest.raises(OutOfPagesError):
                    m.grow(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.requests[rid].num_tokens == n
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.free_pages() == [40, 25] and m.slots.num_free == 5


def test_pools_for_keys_and_values_of_different_widths():
    """A group may cache values narrower (or wider) than its keys, or none at all: the pools then are
    two tensors, pages are counted and poisoned in both, and the bytes per token follow the widths."""
    import torch

    from edgerag_b200.cache.device import DevicePools

    lay = CacheLayout(groups=[KVGroupSpec(2, 3, 16), KVGroupSpec(1, 1, 48, 0, v_head_dim=8), KVGroupSpec(1, 2, 24, 0, v_head_dim=0)],
                      placement=[(0, 0), (1, 0), (0, 1), (2, 0)])
    assert lay.bytes_per_token(2) == 2 * (2 * 3 * 32 + 1 * 1 * 56 + 1 * 2 * 24)
    pools = DevicePools(lay, page_size=4, num_pages=[5, 6, 7], max_requests=2, dtype=torch.float32,
                        device=torch.device("cpu"), poison=True)
    k0, v0 = pools.pages_of(2)
    assert k0.shape == v0.shape == (5, 3, 4, 16) and k0.data_ptr() != v0.data_ptr()
    k1, v1 = pools.pages_of(1)
    assert k1.shape == (6, 1, 4, 48) and v1.shape == (6, 1, 4, 8)
    k2, v2 = pools.pages_of(3)
    assert k2.shape == (7, 2, 4, 24) and v2.shape == (7, 2, 4, 0)
    for t in (k0, v0, k1, v1, k2):
        t.zero_()
    pools.poison_pages([(1, 4), (0, 2), (2, 6)])
    assert torch.isnan(k1[4]).all() and torch.isnan(v1[4]).all() and not torch.isnan(k1[:4]).any()
    assert torch.isnan(k0[2]).all() and torch.isnan(v0[2]).all() and not torch.isnan(v0[3]).any()
    assert torch.isnan(k2[6]).all() and not torch.isnan(k2[:6]).any()
    assert pools.nbytes() == 4 * (5 * 2 * 2 * 3 * 4 * 16 + 6 * 4 * 56 + 7 * 2 * 4 * 24)

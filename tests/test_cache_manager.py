"""The cache manager's bookkeeping: the allocator's contract (the reference's
own five allocator tests, crates/cellm-cache/src/allocator.rs:92-152, and four
page-table tests, crates/cellm-cache/src/pagetable.rs:124-198, restated), and
under random orders of requests: no page lost, held twice or freed twice."""
import random

import pytest
import torch

from cellm_b200.cache import BlockAllocator, CacheError, CacheManager, OutOfPages
from cellm_b200.parts import FixedState, PagedKV


def test_allocator_roundtrip_fifo_exhaustion_and_errors():
    a = BlockAllocator(4)
    assert [a.alloc() for _ in range(4)] == [0, 1, 2, 3] and a.alloc() is None and a.free_count == 0
    a.free(2)
    a.free(0)
    assert a.free_count == 2 and a.is_free(2) and not a.is_free(1)
    assert a.alloc() == 2 and a.alloc() == 0          # first freed, first handed out again
    with pytest.raises(CacheError, match="twice"):
        a.free(1), a.free(1)
    with pytest.raises(CacheError, match="out of range"):
        a.free(9)
    with pytest.raises(CacheError):
        BlockAllocator(0)


def test_alloc_n_is_all_or_nothing():
    a = BlockAllocator(5)
    assert a.alloc_n(3) == [0, 1, 2]
    assert a.alloc_n(3) is None and a.free_count == 2
    assert a.alloc_n(2) == [3, 4] and a.alloc_n(0) == []


def make(pages=8, page=4, slots=3, windows=(0,), extra_state=True):
    needs = [PagedKV(2, 8, w) for w in windows] + ([FixedState((2, 8))] if extra_state else [])
    return CacheManager(needs, [None] * len(needs), page, pages, slots, torch.float32, "cpu")


def test_pages_grow_on_demand_and_map_tokens():
    cm = make()
    cm.add(7)
    assert cm.reserve(7, 1) and list(cm.block_table(7, 0)) == [0]
    cm.commit(7, 1)
    assert cm.reserve(7, 4) and len(cm.block_table(7, 0)) == 1     # still inside the first page
    assert cm.reserve(7, 5) and list(cm.block_table(7, 0)) == [0, 1]
    cm.commit(7, 5)
    assert cm.tokens(7) == 5 and cm.free_pages(0) == 6
    cm.release(7)
    assert cm.free_pages(0) == 8 and cm.free_slots == 3 and cm.live == 0
    with pytest.raises(CacheError):
        cm.tokens(7)


def test_out_of_pages_and_out_of_slots():
    cm = make(pages=2, slots=2)
    cm.add(1)
    assert cm.reserve(1, 8)
    assert not cm.reserve(1, 9)                                     # nothing is taken on failure
    cm.add(2)
    assert not cm.reserve(2, 1)
    with pytest.raises(OutOfPages):
        cm.add(3)
    cm.release(1)
    assert cm.reserve(2, 8)
    with pytest.raises(CacheError):
        cm.commit(2, 9)                                             # more than was reserved
    with pytest.raises(CacheError):
        cm.add(2)                                                   # already live


def test_groups_have_pages_of_their_own_and_windows_give_pages_back():
    cm = make(pages=6, page=4, windows=(0, 6))
    cm.add(1)
    total = 0
    for step in (5, 3, 1, 1, 1, 7, 1, 1):
        total += step
        assert cm.reserve(1, total)
        cm.commit(1, total)
        full, win = cm.block_table(1, 0), cm.block_table(1, 1)
        assert len(full) == len(win) == -(-total // 4) and (full >= 0).all()
        # a page of the windowed group is kept iff a later token can still read one of its keys
        first_needed = max(0, total - 6 + 1)
        for blk, p in enumerate(win):
            assert (p >= 0) == ((blk + 1) * 4 > first_needed), (total, blk, list(win))
    assert cm.free_pages(0) == 6 - 5 and cm.free_pages(1) >= 3
    cm.release(1)
    assert cm.free_pages(0) == cm.free_pages(1) == 6


def test_pages_for_bounds_a_lone_request():
    cm = make(pages=64, page=4, windows=(0, 6))
    assert cm.pages_for(0, 30, 8) == 8
    need = cm.pages_for(1, 200, 8)
    assert need < 50
    cm.add(1)
    total, peak = 0, 0
    while total < 200:
        total = min(200, total + 8)
        assert cm.reserve(1, total)
        peak = max(peak, 64 - cm.free_pages(1))
        cm.commit(1, total)
    assert peak <= need


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page_and_share_none(seed):
    rng = random.Random(seed)
    pages, page, slots = 24, 4, 4
    cm = make(pages=pages, page=page, slots=slots, windows=(0, 10))
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < slots:
            cm.add(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            want = live[rid] + rng.choice([1, 1, 1, 2, 5, 9])
            before = [cm.free_pages(g) for g in (0, 1)]
            if cm.reserve(rid, want):
                cm.commit(rid, want)
                live[rid] = want
            else:
                assert [cm.free_pages(g) for g in (0, 1)] == before
        elif live:
            rid = rng.choice(list(live))
            cm.release(rid)
            del live[rid]
        # invariants: every page is either free or held by exactly one request
        for g in (0, 1):
            held = [p for rid in live for p in cm.block_table(rid, g) if p >= 0]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + cm.free_pages(g) == pages, "a page was lost"
        held_slots = [cm.slot(rid) for rid in live]
        assert len(set(held_slots)) == len(held_slots) and len(held_slots) + cm.free_slots == slots
        for rid, n in live.items():
            assert cm.tokens(rid) == n and len(cm.block_table(rid, 0)) >= -(-n // page)
    for rid in list(live):
        cm.release(rid)
    assert cm.free_pages(0) == cm.free_pages(1) == pages and cm.free_slots == slots


def test_state_slot_is_zeroed_at_admission():
    cm = make(slots=2)
    s = cm.add(1)
    cm.states[0][:, s] = 3.0
    cm.release(1)
    cm.add(2)           # FIFO: the other slot first
    s2 = cm.add(3)
    assert s2 == s and float(cm.states[0][:, s2].abs().max()) == 0.0


def test_bindings_follow_the_order_and_borrowed_caches():
    needs = [FixedState((2, 8)), PagedKV(2, 8, 0), PagedKV(2, 8, 0), None, PagedKV(1, 16, 0)]
    cm = CacheManager(needs, [None, None, None, 1, None], 4, [6, 3], 2, torch.float32, "cpu")
    assert tuple(cm.k_pools[0].shape) == (2, 6, 2, 4, 8) and tuple(cm.k_pools[1].shape) == (1, 3, 1, 4, 16)
    t0, t1 = torch.zeros(1, 2, dtype=torch.int32), torch.zeros(1, 1, dtype=torch.int32)
    b = cm.bindings([t0, t1])
    assert b[0].state is cm.states[0][0].untyped_storage() or b[0].state.shape == (2, 2, 8)
    assert b[1].k.data_ptr() == cm.k_pools[0][0].data_ptr() and b[2].k.data_ptr() == cm.k_pools[0][1].data_ptr()
    assert b[3].k.data_ptr() == b[1].k.data_ptr() and b[3].writes is False and b[1].writes is True
    assert b[4].block_table is t1 and b[4].num_pages == 3
    assert cm.bytes_per_token() == 2 * 4 * (2 * 2 * 8 + 1 * 1 * 16)


def test_requests_of_a_model_without_paged_items_hold_a_slot_only():
    """Layers with fixed-size state alone (no attention anywhere): no page group exists,
    a request of any length fits, and what limits the live requests is the slots."""
    cm = CacheManager([FixedState((2, 8)), FixedState((2, 8))], [None, None], 4, 8, 2, torch.float32, "cpu")
    assert cm.paged_keys == [] and cm.group_pages == [] and cm.k_pools == []
    a, b = cm.add(1), cm.add(2)
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        cm.add(3)
    assert cm.reserve(1, 10_000)
    cm.commit(1, 10_000)
    assert cm.tokens(1) == 10_000
    cm.release(1)
    assert cm.free_slots == 1 and cm.add(3) == a

"""The cache manager on the host: no page lost, held twice or freed twice, under random orders
of requests; window groups give pages back early; state slots."""

from __future__ import annotations

import random

import pytest
import torch
from hypothesis import given, settings, strategies as st

from tinyserve_b200.cache import BlockTable, CacheManager, OutOfPagesError, PageAllocator, RELEASED
from tinyserve_b200.cache.manager import OutOfSlotsError
from tinyserve_b200.parts.base import KVNeed, StateNeed


def test_allocator_basics() -> None:
    a = PageAllocator(4)
    assert a.allocate(2) == [0, 1] and a.num_free == 2
    with pytest.raises(OutOfPagesError):
        a.allocate(3)
    assert a.num_free == 2                                 # all or nothing
    a.share([1])
    a.free([0, 1])
    assert a.owners(1) == 1 and a.owners(0) == 0 and a.num_free == 3
    for bad in ([0], [1, 1], [7]):
        before = (a.num_free, a.owners(1))
        with pytest.raises(ValueError):
            a.free(bad)
        assert (a.num_free, a.owners(1)) == before
    with pytest.raises(ValueError):
        a.share([0])
    a.free([1])
    assert a.allocate(1) == [1]                            # last freed, first reused
    a.check_invariant()


@settings(max_examples=200, deadline=None)
@given(st.lists(st.tuples(st.sampled_from(["alloc", "free", "share"]), st.integers(0, 5)), max_size=60),
       st.integers(1, 12))
def test_allocator_never_loses_or_doubles_a_page(ops, n) -> None:
    a = PageAllocator(n)
    held: list[list[int]] = []
    for op, k in ops:
        if op == "alloc":
            try:
                got = a.allocate(k)
                assert not set(got) & {p for h in held for p in h} or all(a.owners(p) >= 1 for p in got)
                held.append(got)
            except OutOfPagesError:
                assert k > a.num_free
        elif op == "free" and held:
            a.free(held.pop(k % len(held)))
        elif op == "share" and held and held[k % len(held)]:
            pages = held[k % len(held)]
            a.share(pages)
            held.append(list(pages))
        a.check_invariant()
        owners: dict[int, int] = {}
        for h in held:
            for p in h:
                owners[p] = owners.get(p, 0) + 1
        assert all(a.owners(p) == c for p, c in owners.items())
        assert a.num_used == len(owners)
    for h in held:
        a.free(h)
    assert a.num_free == n


def test_block_table_positions_and_window() -> None:
    a = PageAllocator(16)
    t = BlockTable(a, 4)
    t.append(6)
    assert t.pages == [0, 1] and t.slot(5) == 1 * 4 + 1 and t.pages_needed(2) == 0 and t.pages_needed(3) == 1
    with pytest.raises(IndexError):
        t.slot(6)
    w = BlockTable(a, 4, window=5)
    w.append(9)                        # positions 0..8; next query at 9 sees 5..9
    assert w.release_passed() == 1     # page 0 (positions 0..3) is passed; page 1 holds 5..7
    assert w.pages[0] == RELEASED and w.pages_array()[0] == 0 and len(w.live_pages()) == 2
    with pytest.raises(IndexError):
        w.slot(2)
    w.append(8)                        # 17 tokens; next query at 17 sees 13..17
    assert w.release_passed() == 2
    w.release()
    t.release()
    assert a.num_free == 16


def _needs() -> list:
    return [KVNeed(2, 16), KVNeed(2, 16, window=12), KVNeed(2, 16), StateNeed((3, 4)), None, KVNeed(1, 32)]


def test_groups_by_need_and_layout() -> None:
    c = CacheManager(_needs(), page_size=4, num_pages=10, max_requests=3, dtype=torch.float32, device="cpu")
    assert [g.calls for g in c.groups] == [[0, 2], [1], [5]]
    assert c.groups[0].kv.shape == (2, 2, 11, 2, 4, 16)           # calls, k/v, pages + pad, heads, page, dim
    assert c.entries[2].k.data_ptr() == c.groups[0].kv[1, 0].data_ptr()
    assert c.entries[3].state.shape == (3 + 1, 3, 4) and c.entries[4] is None     # one pad slot after the pool
    r = c.new_request()
    assert r.state_slot == 0 and len(r.tables) == 3


def test_state_slots_are_zeroed_and_limited() -> None:
    c = CacheManager(_needs(), page_size=4, num_pages=10, max_requests=2, dtype=torch.float32, device="cpu")
    a = c.new_request()
    c.entries[3].state[a.state_slot] += 5
    b = c.new_request()
    assert not c.can_admit()
    with pytest.raises(OutOfSlotsError):
        c.new_request()
    c.free(a)
    a2 = c.new_request()
    assert a2.state_slot == a.state_slot if a.state_slot >= 0 else True
    assert float(c.entries[3].state[a2.state_slot].abs().sum()) == 0
    c.free(b), c.free(a2)
    with pytest.raises(ValueError):
        c.free(b)


def test_append_is_all_or_nothing_across_groups() -> None:
    c = CacheManager([KVNeed(1, 16), KVNeed(1, 16, window=100)], page_size=4, num_pages=3, max_requests=2,
                     dtype=torch.float32, device="cpu", allocate_memory=False)
    a, b = c.new_request(), c.new_request()
    c.append(a, 8)
    assert c.pages_short(b, 8) == 1 and c.pages_short(None, 4) == 0
    with pytest.raises(OutOfPagesError):
        c.append(b, 8)
    assert all(g.allocator.num_used == 2 for g in c.groups) and b.num_tokens == 0
    c.append(b, 4)
    c.free(a), c.free(b)
    assert all(g.allocator.num_used == 0 for g in c.groups)


@pytest.mark.parametrize("seed", range(20))
def test_random_orders_of_requests_leak_nothing(seed) -> None:
    rng = random.Random(seed)
    c = CacheManager([KVNeed(1, 16), KVNeed(1, 16, window=9), StateNeed((2,))], page_size=4, num_pages=24,
                     max_requests=5, dtype=torch.float32, device="cpu")
    live = []
    for _ in range(300):
        op = rng.random()
        if op < 0.3 and c.can_admit():
            live.append(c.new_request())
        elif op < 0.8 and live:
            r = rng.choice(live)
            n = rng.choice([1, 1, 2, 5, 13])
            if not c.pages_short(r, n):
                c.append(r, n)
                c.release_passed(r)
                assert len(r.tables[1].live_pages()) <= (9 + 13) // 4 + 2
        elif live:
            c.free(live.pop(rng.randrange(len(live))))
        c.check_invariant()
        for g in c.groups:
            held = [p for r in live for p in r.tables[g.index].live_pages()]
            assert len(held) == len(set(held)) == g.allocator.num_used       # none twice, none lost
        assert len({r.state_slot for r in live}) == len(live)
    for r in live:
        c.free(r)
    assert all(g.allocator.num_free == g.num_pages for g in c.groups) and c.state_pool.num_free == 5


def test_a_need_of_another_kind_and_pools_of_different_sizes() -> None:
    """A paged need defined outside the package gets a group, storage and entries of its own
    through its own methods; pools may differ in size group by group; a window group is sized by
    what the requests can hold of it; and a request is refused by what it can ever hold per
    group."""
    from dataclasses import dataclass

    from tinyserve_b200.parts.base import PagedNeed

    @dataclass(frozen=True)
    class OneVector(PagedNeed):
        width: int
        window: int | None = None

        def bytes_per_token(self, element_size):
            return self.width * element_size

        def allocate(self, num_calls, num_pages, page_size, dtype, device):
            return torch.zeros(num_calls, num_pages, page_size, self.width, dtype=dtype, device=device)

        def entry(self, storage, call_in_group, group, page_size):
            return ("mine", group, storage[call_in_group])

    needs = [KVNeed(2, 16), OneVector(24), KVNeed(2, 16, 8), OneVector(24), None]
    c = CacheManager(needs, page_size=4, num_pages=[10, 6, 7], max_requests=3, dtype=torch.float32, device="cpu")
    assert [(g.calls, g.num_pages) for g in c.groups] == [([0], 10), ([1, 3], 6), ([2], 7)]
    assert c.groups[1].kv.shape == (2, 7, 4, 24) and c.entries[3][0] == "mine" and c.entries[3][2].shape == (7, 4, 24)
    assert CacheManager.bytes_per_token(needs, 2) == 2 * (2 * 2 * 16 * 2) + 2 * 24 * 2
    assert c.memory_bytes() == sum(g.kv.numel() * 4 for g in c.groups)
    assert c.capacity_tokens == 6 * 4
    assert c.can_ever_hold(24, 8) and not c.can_ever_hold(25, 8)          # the smallest full group decides
    # one number for all, and the step's token budget known: the window group shrinks to what
    # max_requests requests can hold of it (window 8 + 8 new tokens on pages of 4, one page of slack)
    c = CacheManager(needs, page_size=4, num_pages=100, max_requests=3, dtype=torch.float32, device="cpu",
                     allocate_memory=False, max_step_tokens=8)
    assert [g.num_pages for g in c.groups] == [100, 100, 3 * 5]
    r = c.new_request()
    c.append(r, 8)
    assert [t.num_tokens for t in r.tables] == [8, 8, 8]
    with pytest.raises(TypeError, match="neither a PagedNeed nor a SlotNeed"):
        CacheManager([object()], page_size=4, num_pages=4, max_requests=1, dtype=torch.float32, device="cpu")

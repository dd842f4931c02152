"""The cache manager: page pools for keys and values, and slots for fixed-size state.

The model reports, per call of its run order, what that call keeps between steps
(``KVNeed``, ``StateNeed`` or nothing). Calls with the same need share a **page group**:
one pool of pages, one allocator and, per request, one block table. Groups with different
needs (all positions, a window of them, another head layout) have pages of their own, so a
window group can give pages back early without disturbing the others. Every call of a group
has its own key and value tensors, indexed by the group's page ids:

    kv[call_in_group, 0 = keys / 1 = values, page, kv_head, offset_in_page, head_dim]

so the keys of one (page, kv head) are one contiguous run of ``page_size * head_dim``
elements. One extra page after the pool (``pad_page``) is never handed out; fixed-shape
padding rows may write there.

Requests that hold fixed-size state get one slot id from ``StatePool``; every call with a
``StateNeed`` has a tensor ``[slots, *shape]`` indexed by it, zeroed when the slot is
handed out. An architecture without such calls has an empty pool.

Upstream has one group and no state (src/tinyserve/kv_cache.py:21-50,
src/tinyserve/block_table.py); groups and slots are this framework's own.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import KVCacheEntry, KVNeed, StateCacheEntry, StateNeed
from .allocator import OutOfPagesError, PageAllocator
from .block_table import BlockTable


class OutOfSlotsError(RuntimeError):
    """Every state slot is taken."""


@dataclass
class PageGroup:
    index: int
    need: KVNeed
    page_size: int
    num_pages: int
    calls: list[int]
    allocator: PageAllocator
    kv: torch.Tensor | None = None     # [calls, 2, pages + 1, kv_heads, page_size, head_dim]

    @property
    def pad_page(self) -> int:
        return self.num_pages

    def bytes_per_page(self, element_size: int) -> int:
        return 2 * len(self.calls) * self.need.num_kv_heads * self.page_size * self.need.head_dim * element_size


class StatePool:
    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._used: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfSlotsError(f"all {self.num_slots} state slots are taken")
        s = self._free.pop()
        self._used.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._used:
            raise ValueError(f"free() of a state slot that is not in use: {slot}")
        self._used.remove(slot)
        self._free.append(slot)


@dataclass
class RequestCache:
    """What one live request holds: a block table per page group and maybe a state slot."""

    tables: list[BlockTable]
    state_slot: int = -1
    num_tokens: int = 0
    released: bool = field(default=False)
    uid: int = 0            # unique over the manager's life (object ids may be reused)


class CacheManager:
    def __init__(self, needs: list[KVNeed | StateNeed | None], *, page_size: int, num_pages: int,
                 max_requests: int, dtype: torch.dtype, device: torch.device | str,
                 allocate_memory: bool = True) -> None:
        """``needs`` has one entry per call of the model's run order. ``num_pages`` is the
        size of every page group's pool. ``allocate_memory=False`` keeps the bookkeeping
        only (host-side tests, schedulers driven by a fake model)."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size, self.num_pages = page_size, num_pages
        self.dtype, self.device = dtype, torch.device(device)
        self._next_uid = 0
        self.groups: list[PageGroup] = []
        self.entries: list[KVCacheEntry | StateCacheEntry | None] = [None] * len(needs)
        by_need: dict[KVNeed, PageGroup] = {}
        state_calls: list[tuple[int, StateNeed]] = []
        for call, need in enumerate(needs):
            if isinstance(need, KVNeed):
                g = by_need.get(need)
                if g is None:
                    g = PageGroup(len(self.groups), need, page_size, num_pages, [], PageAllocator(num_pages))
                    by_need[need] = g
                    self.groups.append(g)
                g.calls.append(call)
            elif isinstance(need, StateNeed):
                state_calls.append((call, need))
            elif need is not None:
                raise TypeError(f"call {call}: unknown cache need {need!r}")
        self.state_pool = StatePool(max_requests if state_calls else 0)
        self.has_state = bool(state_calls)
        if allocate_memory:
            for g in self.groups:
                n = g.need
                g.kv = torch.zeros((len(g.calls), 2, num_pages + 1, n.num_kv_heads, page_size, n.head_dim),
                                   dtype=dtype, device=self.device)
                for j, call in enumerate(g.calls):
                    self.entries[call] = KVCacheEntry(g.index, g.kv[j, 0], g.kv[j, 1], page_size)
            for call, need in state_calls:
                state = torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=self.device)
                self.entries[call] = StateCacheEntry(state)

    # ---- sizes
    def memory_bytes(self) -> int:
        total = 0
        for e in self.entries:
            if isinstance(e, KVCacheEntry):
                total += 2 * e.k.numel() * e.k.element_size()
            elif isinstance(e, StateCacheEntry):
                total += e.state.numel() * e.state.element_size()
        return total

    @staticmethod
    def bytes_per_token(needs: list[KVNeed | StateNeed | None], element_size: int) -> int:
        return sum(2 * n.num_kv_heads * n.head_dim * element_size for n in needs if isinstance(n, KVNeed))

    @property
    def utilization(self) -> float:
        if not self.groups:
            return 0.0
        return max(g.allocator.num_used / g.num_pages for g in self.groups)

    # ---- requests
    def new_request(self) -> RequestCache:
        slot = -1
        if self.has_state:
            slot = self.state_pool.allocate()
            for e in self.entries:
                if isinstance(e, StateCacheEntry):
                    e.state[slot].zero_()
        tables = [BlockTable(g.allocator, g.page_size, g.need.window) for g in self.groups]
        self._next_uid += 1
        return RequestCache(tables, slot, uid=self._next_uid)

    def can_admit(self) -> bool:
        return not self.has_state or self.state_pool.num_free > 0

    def pages_short(self, req: RequestCache | None, n: int) -> int:
        """How many pages are lacking, in the worst group, to append ``n`` tokens to ``req``
        (``None`` = a request that holds nothing yet). 0 means it fits."""
        short = 0
        for i, g in enumerate(self.groups):
            if req is None:
                need = (n + g.page_size - 1) // g.page_size
            else:
                need = req.tables[i].pages_needed(n)
            short = max(short, need - g.allocator.num_free)
        return max(short, 0)

    def pages_short_for_all(self, reqs: "list[RequestCache]", n: int) -> int:
        """How many pages are lacking, in the worst group, to append ``n`` tokens to every one
        of ``reqs``. 0 means they all fit."""
        short = 0
        for i, g in enumerate(self.groups):
            need = sum(r.tables[i].pages_needed(n) for r in reqs)
            short = max(short, need - g.allocator.num_free)
        return max(short, 0)

    def pages_for(self, num_tokens: int) -> int:
        """Pages a request of ``num_tokens`` tokens holds at most in any group."""
        return (num_tokens + self.page_size - 1) // self.page_size

    def append(self, req: RequestCache, n: int) -> None:
        """Reserve room for ``n`` more tokens in every group, or in none."""
        if req.released:
            raise ValueError("append() on a request whose cache was freed")
        if len(req.tables) > 1:            # one group alone is all-or-nothing by itself
            short = self.pages_short(req, n)
            if short:
                raise OutOfPagesError(f"{short} pages short for {n} tokens")
        for t in req.tables:
            t.append(n)
        req.num_tokens += n

    def release_passed(self, req: RequestCache) -> int:
        """After a step: give back pages that a window has passed."""
        return sum(t.release_passed() for t in req.tables)

    def free(self, req: RequestCache) -> None:
        if req.released:
            raise ValueError("free() of a request whose cache was already freed")
        for t in req.tables:
            t.release()
        if req.state_slot >= 0:
            self.state_pool.free(req.state_slot)
            req.state_slot = -1
        req.num_tokens = 0
        req.released = True

    def check_invariant(self) -> None:
        for g in self.groups:
            g.allocator.check_invariant()

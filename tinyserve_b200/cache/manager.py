"""The cache manager: page pools for keys and values, and slots for fixed-size state.

The model reports, per cache user (a call of its run order and a mixer of that call's block),
what it keeps between steps: a ``PagedNeed``, a ``SlotNeed`` or nothing (``parts.base``). The
manager serves the two families through their own methods (``allocate``, ``entry``,
``bytes_per_token``), so a need of a new shape is a new subclass and no change here.

Users with equal paged needs share a **page group**: one pool of pages, one allocator and, per
request, one block table. Groups with different needs (all positions, a window of them, another
layout) have pages of their own, so a window group can give pages back early without disturbing
the others, and a pool of its own size: a request never holds more pages of a window group than
its window and one step's tokens cover, so such a group is given only as many pages as
``max_requests`` requests can hold at once (when the step's token budget is known). Every user of
a group has its own part of the group's storage, indexed by the group's page ids; for ``KVNeed``

    kv[call_in_group, 0 = keys / 1 = values, page, kv_head, offset_in_page, head_dim]

so the keys of one (page, kv head) are one contiguous run of ``page_size * head_dim``
elements. One extra page after the pool (``pad_page``) is never handed out; fixed-shape
padding rows may write there.

Requests that hold fixed-size state get one slot id from ``StatePool``; every user with a
``SlotNeed`` has storage ``[slots + 1, ...]`` indexed by it, zeroed when the slot is handed out
(the last row is the pad slot for padding rows). An architecture without such users has an empty
pool.

Upstream has one group and no state (src/tinyserve/kv_cache.py:21-50,
src/tinyserve/block_table.py); groups and slots are this framework's own.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from typing import Any, Sequence

from ..parts.base import CacheNeed, PagedNeed, SlotNeed
from .allocator import OutOfPagesError, PageAllocator
from .block_table import BlockTable


class OutOfSlotsError(RuntimeError):
    """Every state slot is taken."""


@dataclass
class PageGroup:
    index: int
    need: PagedNeed
    page_size: int
    num_pages: int
    calls: list[int]
    allocator: PageAllocator
    kv: torch.Tensor | None = None     # the need's storage; KVNeed: [calls, 2, pages + 1, kv_heads, page_size, head_dim]

    @property
    def pad_page(self) -> int:
        return self.num_pages

    def bytes_per_page(self, element_size: int) -> int:
        return len(self.calls) * self.need.bytes_per_token(element_size) * self.page_size

    def most_pages_of(self, num_tokens: int, step_tokens: int) -> int:
        """The most pages of this group that a request of up to ``num_tokens`` tokens ever holds
        at one time when a step brings it at most ``step_tokens`` tokens: all of its pages, or,
        with a window, those that the window and one step's tokens cover (before the pages the
        window has passed are given back after the step)."""
        pages = -(-num_tokens // self.page_size)
        if self.need.window is not None:
            pages = min(pages, -(-(self.need.window + min(step_tokens, num_tokens)) // self.page_size) + 1)
        return pages


class StatePool:
    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self.pad_slot = num_slots        # a row after the pool, never handed out
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
    def __init__(self, needs: Sequence[CacheNeed | None], *, page_size: int, num_pages: int | Sequence[int],
                 max_requests: int, dtype: torch.dtype, device: torch.device | str,
                 allocate_memory: bool = True, max_step_tokens: int | None = None) -> None:
        """``needs`` has one entry per cache user of the model (``DecoderModel.cache_needs``).
        ``num_pages``: the size of a page pool; one number for all groups, or one per group in the
        order in which their needs first appear (``distinct_paged_needs``). With one number and
        ``max_step_tokens`` (the most tokens a step brings one request) given, a window group gets
        no more pages than ``max_requests`` requests can hold of it. ``allocate_memory=False`` keeps
        the bookkeeping only (host-side tests, schedulers driven by a fake model)."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        distinct = self.distinct_paged_needs(needs)
        if isinstance(num_pages, int):
            sizes = [num_pages] * len(distinct)
            if max_step_tokens is not None:
                for i, need in enumerate(distinct):
                    if need.window is not None:
                        per_request = -(-(need.window + max_step_tokens) // page_size) + 1
                        sizes[i] = min(num_pages, max_requests * per_request)
        else:
            sizes = [int(n) for n in num_pages]
            if len(sizes) != len(distinct):
                raise ValueError(f"{len(sizes)} pool sizes for {len(distinct)} page groups")
        self.page_size = page_size
        self.num_pages = max(sizes, default=int(num_pages) if isinstance(num_pages, int) else 0)
        self.max_step_tokens = max_step_tokens
        self.dtype, self.device = dtype, torch.device(device)
        self._next_uid = 0
        self.groups: list[PageGroup] = []
        self.entries: list[Any] = [None] * len(needs)
        by_need: dict[PagedNeed, PageGroup] = {}
        slot_users: list[tuple[int, SlotNeed]] = []
        for call, need in enumerate(needs):
            if isinstance(need, PagedNeed):
                g = by_need.get(need)
                if g is None:
                    n = sizes[len(self.groups)]
                    g = PageGroup(len(self.groups), need, page_size, n, [], PageAllocator(n))
                    by_need[need] = g
                    self.groups.append(g)
                g.calls.append(call)
            elif isinstance(need, SlotNeed):
                slot_users.append((call, need))
            elif need is not None:
                raise TypeError(f"cache user {call}: {need!r} is neither a PagedNeed nor a SlotNeed")
        self.state_pool = StatePool(max_requests if slot_users else 0)
        self.has_state = bool(slot_users)
        self._slot_storage: list[torch.Tensor] = []
        if allocate_memory:
            for g in self.groups:
                g.kv = g.need.allocate(len(g.calls), g.num_pages + 1, page_size, dtype, self.device)
                for j, call in enumerate(g.calls):
                    self.entries[call] = g.need.entry(g.kv, j, g.index, page_size)
            for call, need in slot_users:
                storage = need.allocate(max_requests + 1, self.device)
                self._slot_storage.append(storage)
                self.entries[call] = need.entry(storage)

    @staticmethod
    def distinct_paged_needs(needs: Sequence[CacheNeed | None]) -> list[PagedNeed]:
        """The paged needs that get a page group each, in the order of the groups."""
        out: list[PagedNeed] = []
        for need in needs:
            if isinstance(need, PagedNeed) and need not in out:
                out.append(need)
        return out

    # ---- sizes
    def memory_bytes(self) -> int:
        storages = [g.kv for g in self.groups if g.kv is not None] + self._slot_storage
        return sum(t.numel() * t.element_size() for t in storages)

    @staticmethod
    def bytes_per_token(needs: Sequence[CacheNeed | None], element_size: int) -> int:
        return sum(n.bytes_per_token(element_size) for n in needs if isinstance(n, PagedNeed))

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
            for storage in self._slot_storage:
                storage[slot].zero_()
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

    def can_ever_hold(self, num_tokens: int, step_tokens: int) -> bool:
        """Whether a request of up to ``num_tokens`` tokens, fed at most ``step_tokens`` a step,
        fits every page group when it has the cache to itself."""
        return all(g.most_pages_of(num_tokens, step_tokens) <= g.num_pages for g in self.groups)

    @property
    def capacity_tokens(self) -> int:
        """Tokens of one request that the smallest group without a window holds."""
        full = [g.num_pages for g in self.groups if g.need.window is None]
        return (min(full) if full else self.num_pages) * self.page_size

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

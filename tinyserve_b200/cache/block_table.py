"""A request's pages in one page group, in position order.

Position ``p`` lives in ``pages[p // page_size]`` at offset ``p % page_size`` (upstream
src/tinyserve/block_table.py:19-89). For a group that only needs a window of the positions,
pages the window has passed are given back early and their entries become ``RELEASED``.
"""

from __future__ import annotations

import numpy as np

from .allocator import PageAllocator

RELEASED = -1


class BlockTable:
    def __init__(self, allocator: PageAllocator, page_size: int, window: int | None = None) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.allocator = allocator
        self.page_size = page_size
        self.window = window
        self.pages: list[int] = []
        self.num_tokens = 0
        self._first_live = 0       # entries before this index are RELEASED
        # int32 mirror of ``pages`` for building device block tables without a Python loop;
        # released entries hold 0 there (a valid page id that the kernels never look at).
        self._mirror = np.zeros(16, dtype=np.int32)

    def pages_needed(self, n: int) -> int:
        """New pages that appending ``n`` tokens would take. Changes nothing."""
        total = self.num_tokens + n
        return (total + self.page_size - 1) // self.page_size - len(self.pages)

    def append(self, n: int) -> None:
        """Reserve room for ``n`` more tokens; all-or-nothing (``OutOfPagesError``)."""
        if n < 0:
            raise ValueError(f"cannot append {n} tokens")
        new = self.allocator.allocate(self.pages_needed(n))
        if new:
            start = len(self.pages)
            self.pages.extend(new)
            self._ensure_mirror(len(self.pages))
            self._mirror[start: len(self.pages)] = new
        self.num_tokens += n

    def _ensure_mirror(self, n: int) -> None:
        if n > self._mirror.shape[0]:
            grown = np.zeros(max(n, 2 * self._mirror.shape[0]), dtype=np.int32)
            grown[: self._mirror.shape[0]] = self._mirror
            self._mirror = grown

    def pages_array(self) -> np.ndarray:
        """``[len(pages)]`` int32 view for the device block table (released entries are 0)."""
        return self._mirror[: len(self.pages)]

    def adopt(self, pages: list[int]) -> None:
        """Start an empty table on full pages another owner already filled (prefix hook)."""
        if self.pages:
            raise ValueError("adopt() needs an empty table")
        self.allocator.share(pages)
        self.pages = list(pages)
        self._ensure_mirror(len(pages))
        self._mirror[: len(pages)] = pages
        self.num_tokens = len(pages) * self.page_size

    def slot(self, pos: int) -> int:
        if not 0 <= pos < self.num_tokens:
            raise IndexError(f"position {pos} not in 0..{self.num_tokens - 1}")
        page = self.pages[pos // self.page_size]
        if page == RELEASED:
            raise IndexError(f"position {pos} lies on a page the window has passed")
        return page * self.page_size + pos % self.page_size

    def release_passed(self) -> int:
        """Give back pages that no later query can see: the next query is at position
        ``num_tokens`` and sees positions above ``num_tokens - window``. Returns how many."""
        if self.window is None:
            return 0
        first_needed = self.num_tokens - self.window + 1     # lowest position still visible
        if first_needed <= 0:
            return 0
        upto = min(first_needed // self.page_size, len(self.pages))
        gone = [p for p in self.pages[self._first_live:upto] if p != RELEASED]
        if gone:
            self.allocator.free(gone)
        for i in range(self._first_live, upto):
            self.pages[i] = RELEASED
            self._mirror[i] = 0
        self._first_live = max(self._first_live, upto)
        return len(gone)

    def live_pages(self) -> list[int]:
        return [p for p in self.pages if p != RELEASED]

    def release(self) -> None:
        live = self.live_pages()
        if live:
            self.allocator.free(live)
        self.pages = []
        self.num_tokens = 0
        self._first_live = 0

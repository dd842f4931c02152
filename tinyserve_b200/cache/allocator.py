"""Page allocator: which page ids of a pool are free and how many owners each used page has.

Bookkeeping only; it never touches a tensor. Semantics after upstream
src/tinyserve/block_allocator.py:38-121: ``allocate(n)`` is all-or-nothing and raises
``OutOfPagesError`` without changing anything; ``share`` adds an owner to pages in use (the
hook for prefix sharing); ``free`` drops one owner and returns a page to the pool when its
last owner lets go; a double free, an unknown id or a duplicate id in one call is a
``ValueError`` that changes nothing. Freed pages are reused last-freed-first.
"""

from __future__ import annotations


class OutOfPagesError(RuntimeError):
    """More pages were asked for than are free."""


class PageAllocator:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # a stack; page 0 is handed out first
        self._owners: dict[int, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return len(self._owners)

    def owners(self, page: int) -> int:
        return self._owners.get(page, 0)

    def allocate(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise OutOfPagesError(f"asked for {n} pages, {len(self._free)} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._owners[p] = 1
        return pages

    def _check(self, pages: list[int], what: str) -> None:
        if len(set(pages)) != len(pages):
            raise ValueError(f"duplicate page ids in {what}(): {pages}")
        for p in pages:
            if p not in self._owners:
                raise ValueError(f"{what}() of a page that is not in use: {p}")

    def share(self, pages: list[int]) -> None:
        self._check(pages, "share")
        for p in pages:
            self._owners[p] += 1

    def free(self, pages: list[int]) -> None:
        self._check(pages, "free")
        for p in pages:
            self._owners[p] -= 1
            if self._owners[p] == 0:
                del self._owners[p]
                self._free.append(p)

    def check_invariant(self) -> None:
        """Every id is free or owned, never both, never twice."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        assert not (free & set(self._owners)), "a page is both free and owned"
        assert free | set(self._owners) == set(range(self.num_pages)), "a page is lost"
        assert all(c >= 1 for c in self._owners.values())

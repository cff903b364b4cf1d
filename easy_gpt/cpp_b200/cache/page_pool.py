"""Allocator of page ids for one cache group: a LIFO stack of free ids, so that
a page given back is the next one handed out (a small pool reuses ids at once).
Pure host code; it owns no memory."""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Not enough free pages; nothing was changed."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # page 0 is handed out first
        self._held = [False] * num_pages
        self.high_water = 0
        self.total_allocated = 0      # pages handed out over the pool's life (> num_pages: ids were used again)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.total_allocated += n
        self.high_water = max(self.high_water, self.used_count)
        return out

    def free(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} is freed twice")
            self._held[p] = False
        # pushed in reverse so that the lowest id of the batch comes out first again
        for p in reversed(pages):
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free once or held once."""
        free = set(self._free)
        assert len(free) == len(self._free), "a page is on the free list twice"
        for p in range(self.num_pages):
            assert self._held[p] != (p in free), f"page {p} is lost or both held and free"

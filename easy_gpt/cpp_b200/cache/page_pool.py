"""Allocator of page ids for one cache group: a LIFO stack of free ids, so that
a page given back is the next one handed out (a small pool reuses ids at once).
The pool itself is host C++ (``csrc/host/page_pool.hpp``); this class is its face
in Python.  It owns no memory of the cache."""
from __future__ import annotations

import ctypes
from typing import List

import numpy as np

from .. import host


class OutOfPages(RuntimeError):
    """Not enough free pages; nothing was changed."""


class PagePool:
    def __init__(self, num_pages: int, _borrowed=None):
        """``_borrowed``: (handle, owner) of a pool that lives inside a cache's bookkeeping."""
        self._lib = host.library()
        if _borrowed is not None:
            self._handle, self._owner = _borrowed
            self._owned = False
        else:
            if num_pages <= 0:
                raise ValueError("a page pool needs at least one page")
            self._handle = self._lib.egh_pool_create(int(num_pages))
            self._owner, self._owned = None, True
        self.num_pages = int(self._lib.egh_pool_stat(self._handle, 0))

    def __del__(self):
        if getattr(self, "_owned", False) and self._handle:
            self._lib.egh_pool_destroy(self._handle)
            self._handle = None

    @property
    def free_count(self) -> int:
        return int(self._lib.egh_pool_stat(self._handle, 1))

    @property
    def used_count(self) -> int:
        return self.num_pages - self.free_count

    @property
    def high_water(self) -> int:
        return int(self._lib.egh_pool_stat(self._handle, 2))

    @property
    def total_allocated(self) -> int:
        """Pages handed out over the pool's life (more than num_pages: ids were used again)."""
        return int(self._lib.egh_pool_stat(self._handle, 3))

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        out = np.empty(max(n, 1), dtype=np.int32)
        rc = self._lib.egh_pool_alloc(self._handle, int(n), out.ctypes.data)
        if rc == host.OUT_OF_PAGES:
            raise OutOfPages(f"{n} pages wanted, {self.free_count} free of {self.num_pages}")
        return out[:n].tolist()

    def free(self, pages) -> None:
        """All of ``pages`` or, with an exception, none."""
        arr = np.ascontiguousarray(list(pages), dtype=np.int32)
        bad = ctypes.c_int(0)
        rc = self._lib.egh_pool_free(self._handle, arr.ctypes.data, int(arr.size), ctypes.byref(bad))
        if rc == host.NOT_OF_POOL:
            raise ValueError(f"page {bad.value} is not of this pool")
        if rc == host.FREED_TWICE:
            raise ValueError(f"page {bad.value} is freed twice")

    def check(self) -> None:
        """Every page is either free once or held once."""
        assert self._lib.egh_pool_check(self._handle) == host.OK, "a page is lost, on the free list twice, or both held and free"

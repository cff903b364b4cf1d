"""The cache manager: paged keys/values with a block table per request, one pool
per *group* of caches with the same needs, and slots for per-request state of
fixed size.

Each run entry of a model that writes a cache declares what it needs
(``PagedKVNeed`` or ``StateNeed``).  Caches whose need is identical (KV heads,
head size, window) form a group: they share one page pool and one block table,
and page id p addresses the same page in each of them.  A group that keeps all
keys holds ceil(len / page_size) pages per request; a group with a window gives
a page back as soon as every position in it has left the window of all tokens
still to come.  When a request ends, everything it holds is given back.

Memory of a group: one tensor [caches, pages, 2 (k, v), kv_heads, page_size,
head_dim] in the engine's dtype.  State: one tensor [slots, *shape] (of the dtype the
need names) per cache that asked for it, zeroed when a request takes the slot.

(The reference has no pages: its per-sample caches grow by concatenation,
src/models/self_attn.cpp:369-389, or by doubling, src/cuda/ops/self_attn_detail.cuh:951-1022,
and it hands attention a padded copy of all of them each step,
src/models/cache_batching.cpp:25-81.  Slots are its ``free_slots_`` stack,
src/continuous_batch_server.cpp:44-47.)

All bookkeeping is host code (C++, ``csrc/host/cache_core.hpp``; this module is its
face in Python and owns the device tensors) and runs without a GPU (device=None
allocates no tensors).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .. import host
from ..parts.base import CacheView, PagedKVNeed, StateNeed
from .page_pool import OutOfPages, PagePool


class OutOfSlots(RuntimeError):
    pass


class CacheGroup:
    """One group of caches with the same needs: its page pool and block tables live in the C++
    bookkeeping; ``tables`` is a view of them ([slots, max pages per request], -1 where no page is held)."""

    def __init__(self, index: int, need: PagedKVNeed, cache_ids: List[int], page_size: int, pool: PagePool,
                 tables: np.ndarray, max_pages_per_request: int):
        self.index = index
        self.need = need
        self.cache_ids = cache_ids
        self.page_size = page_size
        self.pool = pool
        self.max_pages_per_request = max_pages_per_request
        self.tables = tables
        self.kv: Optional[torch.Tensor] = None
        self.scratch_page = -1

    @property
    def window(self) -> Optional[int]:
        return self.need.window

    def first_needed_page(self, length: int) -> int:
        """Lowest logical page that a token at position >= length can still see."""
        if self.window is None:
            return 0
        first_key = max(0, length - self.window + 1)
        return first_key // self.page_size

    def bytes_per_token(self, element_size: int) -> int:
        return len(self.cache_ids) * 2 * self.need.num_kv_heads * self.need.head_dim * element_size


class CacheManager:
    def __init__(self, needs: Mapping[int, object], page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: int, device=None, dtype: torch.dtype = torch.float32):
        """needs: cache id -> PagedKVNeed | StateNeed | None.  num_pages: pages of every group's pool."""
        if page_size <= 0 or max_slots <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_slots and max_tokens_per_request must be positive")
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_pages_per_request = -(-max_tokens_per_request // page_size)
        self.device = device
        self.dtype = dtype
        self._lib = host.library()
        self.core = self._lib.egh_cache_create(page_size, max_slots, self.max_pages_per_request)
        self.groups: List[CacheGroup] = []
        self.group_of_cache: Dict[int, int] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self._state_needs: Dict[int, StateNeed] = {}
        by_need: Dict[PagedKVNeed, CacheGroup] = {}
        for cache_id in sorted(needs):
            need = needs[cache_id]
            if isinstance(need, PagedKVNeed):
                g = by_need.get(need)
                if g is None:
                    index = self._lib.egh_cache_add_group(self.core, num_pages, -1 if need.window is None else int(need.window))
                    pool = PagePool(num_pages, _borrowed=(self._lib.egh_cache_group_pool(self.core, index), self))
                    tables = np.ctypeslib.as_array(self._lib.egh_cache_group_table(self.core, index),
                                                   shape=(max_slots, self.max_pages_per_request))
                    g = CacheGroup(index, need, [], page_size, pool, tables, self.max_pages_per_request)
                    by_need[need] = g
                    self.groups.append(g)
                g.cache_ids.append(cache_id)
                self.group_of_cache[cache_id] = g.index
            elif isinstance(need, StateNeed):
                self._state_needs[cache_id] = need
            elif need is not None:
                raise TypeError(f"cache {cache_id}: unknown need {need!r}")
        # requests are known to the bookkeeping by a 64-bit handle: a non-negative int is its own handle
        # (the scheduler's request ids), anything else gets a negative one
        self._handles: Dict[Hashable, int] = {}
        self._named: Dict[int, Hashable] = {}
        self._next_named = -1
        self._needed = (ctypes.c_int * max(1, len(self.groups)))()
        self._info = (ctypes.c_int * 3)()
        self._fresh = (ctypes.c_int * max_slots)()
        if device is not None:
            for g in self.groups:
                # one page beyond the pool (id num_pages): rows that pad a captured batch write there
                g.scratch_page = g.pool.num_pages
                g.kv = torch.zeros((len(g.cache_ids), g.pool.num_pages + 1, 2, g.need.num_kv_heads, page_size, g.need.head_dim),
                                   device=device, dtype=dtype)
            for cache_id, need in self._state_needs.items():
                # one slot more than requests can take: the scratch slot that padding rows of a captured batch use
                self.state[cache_id] = torch.zeros((max_slots + 1, *need.shape), device=device, dtype=getattr(torch, need.dtype))

    def __del__(self):
        core = getattr(self, "core", None)
        if core:
            self.core = None
            for g in self.groups:
                g.tables = None            # the views die with the memory they look at
            self._lib.egh_cache_destroy(core)

    # -- handles -------------------------------------------------------------
    def handle(self, rid, create: bool = False) -> Optional[int]:
        """The bookkeeping's 64-bit name of a request (None: unknown and not to be created)."""
        if isinstance(rid, (int, np.integer)) and not isinstance(rid, bool) and 0 <= int(rid) < (1 << 62):
            return int(rid)
        h = self._handles.get(rid)
        if h is None and create:
            h = self._next_named
            self._next_named -= 1
            self._handles[rid] = h
            self._named[h] = rid
        return h

    def _live_handle(self, rid) -> int:
        h = self.handle(rid)
        if h is None or self._lib.egh_cache_query(self.core, h, 0) < 0:
            raise KeyError(rid)
        return h

    def _forget(self, rid, h: int) -> None:
        if h < 0:
            self._handles.pop(rid, None)
            self._named.pop(h, None)

    # -- requests -----------------------------------------------------------
    def has_request(self, rid) -> bool:
        h = self.handle(rid)
        return h is not None and self._lib.egh_cache_query(self.core, h, 0) >= 0

    def live_requests(self) -> List[object]:
        buf = (ctypes.c_longlong * self.max_slots)()
        n = self._lib.egh_cache_live(self.core, buf, self.max_slots)
        return [self._named.get(h, h) for h in sorted(buf[:n], key=lambda h: (h < 0, abs(h)))]

    def free_slot_count(self) -> int:
        return int(self._lib.egh_cache_free_slots(self.core))

    def begin_request(self, rid) -> int:
        known = self.handle(rid) is not None
        h = self.handle(rid, create=True)
        slot = self._lib.egh_cache_begin(self.core, h)
        if slot == host.ALREADY_LIVE:
            raise KeyError(f"request {rid!r} is already live")
        if slot == host.OUT_OF_SLOTS:
            if not known:
                self._forget(rid, h)
            raise OutOfSlots(f"all {self.max_slots} request slots are taken")
        self.zero_fresh_state()
        return int(slot)

    def zero_state(self, slot: int) -> None:
        """A request that takes a slot starts from zeroed per-request state."""
        for t in self.state.values():
            t[slot].zero_()

    def zero_fresh_state(self) -> None:
        """Clears the state of every slot that a request has taken since the last call, whoever began
        the request (this class, the step's reservation or the scheduler, which all begin requests in
        the C++ bookkeeping).  The step function calls it before every forward pass, captured or not,
        so a request never sees what the slot's former owner left (a preempted request that comes back
        starts from zero too: its tokens are computed again)."""
        n = self._lib.egh_cache_take_fresh(self.core, self._fresh, self.max_slots)
        if self.state:
            for slot in self._fresh[:n]:
                self.zero_state(slot)

    def slot_of(self, rid) -> int:
        return int(self._lib.egh_cache_query(self.core, self._live_handle(rid), 0))

    def length_of(self, rid) -> int:
        return int(self._lib.egh_cache_query(self.core, self._live_handle(rid), 1))

    def pages_needed(self, rid, new_tokens: int) -> Dict[int, int]:
        """Pages each group would have to hand out so that ``new_tokens`` more tokens fit."""
        self._lib.egh_cache_pages_needed(self.core, self._live_handle(rid), int(new_tokens), self._needed)
        return {g.index: int(self._needed[g.index]) for g in self.groups}

    def can_reserve(self, rid, new_tokens: int, spare: int = 0) -> bool:
        return self._lib.egh_cache_can_reserve(self.core, self._live_handle(rid), int(new_tokens), int(spare)) == 1

    def reserve(self, rid, new_tokens: int) -> None:
        """Pages for positions length .. length+new_tokens-1 in every group, or
        ``OutOfPages`` with nothing changed."""
        rc = self._lib.egh_cache_reserve(self.core, self._live_handle(rid), int(new_tokens), self._info)
        if rc == host.TOO_LONG:
            raise OutOfPages(f"request {rid!r} would hold {self.length_of(rid) + new_tokens} tokens; a request may hold at most "
                             f"{self.max_pages_per_request * self.page_size}")
        if rc == host.OUT_OF_PAGES:
            raise OutOfPages(f"group {self._info[0]}: {self._info[1]} pages wanted for request {rid!r}, {self._info[2]} free")
        if rc != host.OK:
            raise RuntimeError(f"cache bookkeeping: reserve failed with status {rc}")

    def commit(self, rid, new_tokens: int) -> None:
        """The step has written ``new_tokens`` more tokens.  Pages that no coming
        token can see any more (a window has passed them) are given back."""
        rc = self._lib.egh_cache_commit(self.core, self._live_handle(rid), int(new_tokens))
        if rc == host.EXCEEDS_RESERVED:
            raise ValueError(f"request {rid!r}: commit of {new_tokens} tokens exceeds what was reserved")
        if rc != host.OK:
            raise RuntimeError(f"cache bookkeeping: commit failed with status {rc}")

    def end_request(self, rid) -> None:
        h = self._live_handle(rid)
        rc = self._lib.egh_cache_end(self.core, h)
        if rc != host.OK:
            raise RuntimeError(f"cache bookkeeping: ending request {rid!r} failed with status {rc}")
        self._forget(rid, h)

    def reset(self) -> None:
        for rid in self.live_requests():
            self.end_request(rid)

    # -- what a step needs ---------------------------------------------------
    def slot_positions(self, group: int, rid, start: int, count: int) -> np.ndarray:
        """Physical cache positions (page * page_size + offset) of the request's
        logical positions start .. start+count-1."""
        out = np.empty(max(count, 1), dtype=np.int32)
        rc = self._lib.egh_cache_slot_positions(self.core, group, self._live_handle(rid), int(start), int(count), out.ctypes.data)
        if rc == host.NO_PAGE:
            raise ValueError(f"request {rid!r}: a position in {start}..{start + count - 1} has no page in group {group}")
        return out[:count]

    def table_rows(self, group: int, rids: Sequence, width: int) -> np.ndarray:
        g = self.groups[group]
        slots = [self.slot_of(r) for r in rids]
        return g.tables[slots, :width]

    def view(self, cache_id: int, writes: bool = True) -> CacheView:
        if cache_id in self.group_of_cache:
            g = self.groups[self.group_of_cache[cache_id]]
            if g.kv is None:
                return CacheView(group=g.index, writes=writes)
            layer = g.kv[g.cache_ids.index(cache_id)]
            return CacheView(group=g.index, k=layer[:, 0], v=layer[:, 1], writes=writes)
        if cache_id in self.state:
            return CacheView(state=self.state[cache_id], writes=writes)
        return CacheView(writes=writes)

    # -- accounting ------------------------------------------------------------
    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.free_count

    def kv_bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(es) for g in self.groups)

    def check(self) -> None:
        """No page lost, none held twice: the pages in all block tables are exactly
        the pages the pools consider held; free slots hold nothing."""
        why = ctypes.create_string_buffer(256)
        rc = self._lib.egh_cache_check(self.core, why, 256)
        assert rc == host.OK, why.value.decode()

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
head_dim] in the engine's dtype.  State: one float32 tensor [slots, *shape] per
cache that asked for it, zeroed when a request takes the slot.

(The reference has no pages: its per-sample caches grow by concatenation,
src/models/self_attn.cpp:369-389, or by doubling, src/cuda/ops/self_attn_detail.cuh:951-1022,
and it hands attention a padded copy of all of them each step,
src/models/cache_batching.cpp:25-81.  Slots are its ``free_slots_`` stack,
src/continuous_batch_server.cpp:44-47.)

All bookkeeping is host code and runs without a GPU (device=None allocates no
tensors).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheView, PagedKVNeed, StateNeed
from .page_pool import OutOfPages, PagePool


class OutOfSlots(RuntimeError):
    pass


@dataclass
class _Request:
    slot: int
    length: int = 0                                        # tokens committed to the cache
    reserved: int = 0                                      # tokens for which pages exist (>= length)
    first_live_page: Dict[int, int] = field(default_factory=dict)   # per group: logical pages below were given back


class CacheGroup:
    def __init__(self, index: int, need: PagedKVNeed, cache_ids: List[int], page_size: int, num_pages: int,
                 max_slots: int, max_pages_per_request: int):
        self.index = index
        self.need = need
        self.cache_ids = cache_ids
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.max_pages_per_request = max_pages_per_request
        # host block tables by slot; -1 where no page is held
        self.tables = np.full((max_slots, max_pages_per_request), -1, dtype=np.int32)
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
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_pages_per_request = -(-max_tokens_per_request // page_size)
        self.device = device
        self.dtype = dtype
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
                    g = CacheGroup(len(self.groups), need, [], page_size, num_pages, max_slots, self.max_pages_per_request)
                    by_need[need] = g
                    self.groups.append(g)
                g.cache_ids.append(cache_id)
                self.group_of_cache[cache_id] = g.index
            elif isinstance(need, StateNeed):
                self._state_needs[cache_id] = need
            elif need is not None:
                raise TypeError(f"cache {cache_id}: unknown need {need!r}")
        self._free_slots: List[int] = list(range(max_slots - 1, -1, -1))     # slot 0 first
        self._requests: Dict[object, _Request] = {}
        if device is not None:
            for g in self.groups:
                # one page beyond the pool (id num_pages): rows that pad a captured batch write there
                g.scratch_page = g.pool.num_pages
                g.kv = torch.zeros((len(g.cache_ids), g.pool.num_pages + 1, 2, g.need.num_kv_heads, page_size, g.need.head_dim),
                                   device=device, dtype=dtype)
            for cache_id, need in self._state_needs.items():
                self.state[cache_id] = torch.zeros((max_slots, *need.shape), device=device, dtype=torch.float32)

    # -- requests -----------------------------------------------------------
    def has_request(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self) -> List[object]:
        return list(self._requests)

    def free_slot_count(self) -> int:
        return len(self._free_slots)

    def begin_request(self, rid) -> int:
        if rid in self._requests:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_slots} request slots are taken")
        slot = self._free_slots.pop()
        self._requests[rid] = _Request(slot, first_live_page={g.index: 0 for g in self.groups})
        for t in self.state.values():
            t[slot].zero_()
        return slot

    def slot_of(self, rid) -> int:
        return self._requests[rid].slot

    def length_of(self, rid) -> int:
        return self._requests[rid].length

    def pages_needed(self, rid, new_tokens: int) -> Dict[int, int]:
        """Pages each group would have to hand out so that ``new_tokens`` more tokens fit."""
        r = self._requests[rid]
        target = r.length + new_tokens
        out = {}
        for g in self.groups:
            have = -(-r.reserved // g.page_size)
            want = -(-target // g.page_size)
            out[g.index] = max(0, want - have)
        return out

    def can_reserve(self, rid, new_tokens: int, spare: int = 0) -> bool:
        r = self._requests[rid]
        if -(-(r.length + new_tokens) // self.page_size) > self.max_pages_per_request:
            return False
        return all(self.groups[gi].pool.free_count - spare >= n for gi, n in self.pages_needed(rid, new_tokens).items())

    def reserve(self, rid, new_tokens: int) -> None:
        """Pages for positions length .. length+new_tokens-1 in every group, or
        ``OutOfPages`` with nothing changed."""
        r = self._requests[rid]
        target = r.length + new_tokens
        if -(-target // self.page_size) > self.max_pages_per_request:
            raise OutOfPages(f"request {rid!r} would hold {target} tokens; a request may hold at most "
                             f"{self.max_pages_per_request * self.page_size}")
        needed = self.pages_needed(rid, new_tokens)
        for gi, n in needed.items():
            if self.groups[gi].pool.free_count < n:
                raise OutOfPages(f"group {gi}: {n} pages wanted for request {rid!r}, "
                                 f"{self.groups[gi].pool.free_count} free")
        for gi, n in needed.items():
            g = self.groups[gi]
            have = -(-r.reserved // g.page_size)
            pages = g.pool.alloc(n)
            g.tables[r.slot, have:have + n] = pages
        r.reserved = max(r.reserved, target)

    def commit(self, rid, new_tokens: int) -> None:
        """The step has written ``new_tokens`` more tokens.  Pages that no coming
        token can see any more (a window has passed them) are given back."""
        r = self._requests[rid]
        if r.length + new_tokens > r.reserved:
            raise ValueError(f"request {rid!r}: commit of {new_tokens} tokens exceeds what was reserved")
        r.length += new_tokens
        for g in self.groups:
            first = g.first_needed_page(r.length)
            old = r.first_live_page[g.index]
            if first > old:
                row = g.tables[r.slot]
                g.pool.free([int(p) for p in row[old:first]])
                row[old:first] = -1
                r.first_live_page[g.index] = first

    def end_request(self, rid) -> None:
        r = self._requests.pop(rid)
        for g in self.groups:
            row = g.tables[r.slot]
            held = row[row >= 0]
            g.pool.free([int(p) for p in held])
            row[:] = -1
        self._free_slots.append(r.slot)

    def reset(self) -> None:
        for rid in list(self._requests):
            self.end_request(rid)

    # -- what a step needs ---------------------------------------------------
    def slot_positions(self, group: int, rid, start: int, count: int) -> np.ndarray:
        """Physical cache positions (page * page_size + offset) of the request's
        logical positions start .. start+count-1."""
        g = self.groups[group]
        r = self._requests[rid]
        pos = np.arange(start, start + count, dtype=np.int64)
        pages = g.tables[r.slot, pos // g.page_size].astype(np.int64)
        if (pages < 0).any():
            raise ValueError(f"request {rid!r}: a position in {start}..{start + count - 1} has no page in group {group}")
        return (pages * g.page_size + pos % g.page_size).astype(np.int32)

    def table_rows(self, group: int, rids: Sequence, width: int) -> np.ndarray:
        g = self.groups[group]
        slots = [self._requests[r].slot for r in rids]
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
        the pages the pools consider held."""
        for g in self.groups:
            g.pool.check()
            held = g.tables[g.tables >= 0]
            assert len(held) == len(set(held.tolist())), f"group {g.index}: a page is in two places of the block tables"
            assert len(held) == g.pool.used_count, f"group {g.index}: {g.pool.used_count} pages held, {len(held)} in tables"
            live_slots = {r.slot for r in self._requests.values()}
            for s in range(self.max_slots):
                if s not in live_slots:
                    assert (g.tables[s] < 0).all(), f"group {g.index}: free slot {s} still holds pages"
        assert len(set(self._free_slots)) == len(self._free_slots)
        assert len(self._free_slots) + len(self._requests) == self.max_slots

"""The step function: one batch of (request, its next tokens) through the model.

A batch is any mix of prompt portions and single decoded tokens, cut anywhere.
``StepRunner.run`` reserves cache pages for the new tokens, packs the batch's
metadata into one pinned host buffer, copies it to the device once, runs the
model over exactly the tokens it was given (reading everything earlier from the
cache) and returns float32 logits at the wanted places, in the order of the
entries and of each entry's ``want``.

(The reference has two entry points that never mix, one for padded prompts and
one for single tokens, src/models/gpt_model.cpp:375-419, and computes logits at
every position, :203-211.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheManager
from ..parts.base import GroupTables, StepContext
from .model import Model


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # indices into ``tokens`` whose logits are asked for


class StepError(RuntimeError):
    pass


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    def __init__(self, model: Model, page_size: int, num_pages: int, max_slots: int,
                 max_tokens_per_request: Optional[int] = None, use_graphs: bool = True):
        self.model = model
        self.device = model.device
        max_tokens_per_request = max_tokens_per_request or min(model.spec.max_positions, num_pages * page_size)
        self.cache = CacheManager(model.cache_needs(), page_size, num_pages, max_slots, max_tokens_per_request,
                                  device=model.device, dtype=model.dtype)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # pinned staging buffers in a ring: a buffer is rewritten only after the copy
        # that read it has finished (its event), so steps need not synchronise
        self._ring: List[Optional[torch.Tensor]] = [None] * 4
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._ring_next = 0
        self._dev: Optional[torch.Tensor] = None
        self.steps_run = 0
        self.use_graphs = use_graphs and model.capturable
        self._graphs: Dict[int, object] = {}
        self._signature_graphs: Dict[tuple, object] = {}
        self._graph_pool = None
        self._signature_seen: Dict[tuple, int] = {}
        self.graph_replays = 0

    # -- request lifetime -------------------------------------------------------
    def end(self, request) -> None:
        if self.cache.has_request(request):
            self.cache.end_request(request)

    # -- one step -----------------------------------------------------------------
    def _buffers(self, n_ints: int):
        i = self._ring_next
        self._ring_next = (i + 1) % len(self._ring)
        if self._ring_events[i] is not None:
            self._ring_events[i].synchronize()
        cap = max(1024, 1 << (n_ints - 1).bit_length())
        if self._ring[i] is None or self._ring[i].numel() < n_ints:
            self._ring[i] = torch.empty(cap, dtype=torch.int32).pin_memory()
        if self._dev is None or self._dev.numel() < n_ints:
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return i, self._ring[i], self._dev

    def build_context(self, entries: Sequence[StepEntry]):
        """Reserves pages and packs the batch.  Returns (StepContext, logit_rows tensor or None)."""
        cache = self.cache
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
        started = []
        try:
            for e in entries:
                if not cache.has_request(e.request):
                    cache.begin_request(e.request)
                    started.append(e.request)
            # all-or-nothing over the batch: check first, then take
            spare: Dict[int, int] = {g.index: 0 for g in cache.groups}
            for e in entries:
                for gi, n in cache.pages_needed(e.request, len(e.tokens)).items():
                    spare[gi] += n
            for g in cache.groups:
                if spare[g.index] > g.pool.free_count:
                    from ..cache.page_pool import OutOfPages
                    raise OutOfPages(f"group {g.index}: the step needs {spare[g.index]} new pages, "
                                     f"{g.pool.free_count} are free")
            for e in entries:
                cache.reserve(e.request, len(e.tokens))
        except Exception:
            for r in started:
                cache.end_request(r)
            raise

        n = len(entries)
        counts = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        T = int(counts.sum())
        starts = np.zeros(n + 1, dtype=np.int32)
        starts[1:] = np.cumsum(counts)
        context = np.array([cache.length_of(e.request) for e in entries], dtype=np.int32)
        slots = np.array([cache.slot_of(e.request) for e in entries], dtype=np.int32)
        token_seq = np.repeat(np.arange(n, dtype=np.int32), counts)
        positions = (np.arange(T, dtype=np.int32) - np.repeat(starts[:-1], counts) + np.repeat(context, counts)).astype(np.int32)
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if token_ids.min() < -(1 << 31) or token_ids.max() >= (1 << 31):
            raise StepError("token ids do not fit 32 bits")
        rows = [int(starts[i]) + int(w) for i, e in enumerate(entries) for w in e.want]
        R = len(rows)
        total_len = context.astype(np.int64) + counts
        width = {g.index: int(-(-int(total_len.max()) // g.page_size)) for g in cache.groups}

        tiles, small = kernels.query_tiles_of(starts, counts)
        layout = [("token_ids", T), ("positions", T), ("token_seq", T), ("seq_starts", n + 1), ("seq_context", n),
                  ("seq_slots", n), ("logit_rows", R), ("query_tiles", 3 * len(tiles)), ("small_tokens", len(small))]
        for g in cache.groups:
            layout += [(f"slot_map{g.index}", T), (f"table{g.index}", n * width[g.index])]
        offsets, off = {}, 0
        for name, size in layout:
            offsets[name] = (off, size)
            off += _pad4(size)
        ring_index, host, dev = self._buffers(off)
        hv = host.numpy()

        def put(name, arr):
            o, size = offsets[name]
            hv[o:o + size] = arr

        put("token_ids", token_ids.astype(np.int32))
        put("positions", positions)
        put("token_seq", token_seq)
        put("seq_starts", starts)
        put("seq_context", context)
        put("seq_slots", slots)
        put("logit_rows", np.asarray(rows, dtype=np.int32))
        put("query_tiles", np.asarray(tiles, dtype=np.int32).reshape(-1))
        put("small_tokens", np.asarray(small, dtype=np.int32))
        rids = [e.request for e in entries]
        for g in cache.groups:
            sm = np.concatenate([cache.slot_positions(g.index, e.request, int(context[i]), int(counts[i]))
                                 for i, e in enumerate(entries)])
            put(f"slot_map{g.index}", sm)
            put(f"table{g.index}", cache.table_rows(g.index, rids, width[g.index]).reshape(-1))
        dev[:off].copy_(host[:off], non_blocking=True)
        if self._ring_events[ring_index] is None:
            self._ring_events[ring_index] = torch.cuda.Event()
        self._ring_events[ring_index].record()

        def view(name):
            o, size = offsets[name]
            return dev[o:o + size]

        ctx = StepContext(
            dtype=self.model.dtype, device=self.device, num_tokens=T, num_seqs=n,
            token_ids=view("token_ids"), positions=view("positions"), token_seq=view("token_seq"),
            seq_starts=view("seq_starts"), seq_context=view("seq_context"), seq_slots=view("seq_slots"),
            status=self.status,
            groups={g.index: GroupTables(g.page_size, view(f"table{g.index}").view(n, width[g.index]),
                                         view(f"slot_map{g.index}")) for g in cache.groups},
            host_seq_starts=starts.tolist(), host_seq_context=context.tolist(), host_seq_slots=slots.tolist(),
            max_query_len=int(counts.max()), max_context_len=int(total_len.max()),
            all_decode=bool((counts == 1).all()),
            query_tiles=view("query_tiles").view(len(tiles), 3) if tiles else None,
            small_tokens=view("small_tokens") if tiles and small else None,
        )
        return ctx, (view("logit_rows") if R else None)

    def run(self, entries: Sequence[StepEntry], check: bool = True, commit: bool = True) -> Optional[torch.Tensor]:
        """Logits [wanted, vocab] float32 on the device (None if nothing is wanted).
        With ``check`` the device status word is read back (a synchronisation) and
        a complaint of a kernel becomes an exception.  With ``commit`` the requests'
        cached lengths advance here; a scheduler that keeps its own count passes False
        and calls ``cache.commit`` itself."""
        captured, logits = self._run_captured(entries) if self.use_graphs else (False, None)
        if not captured:
            ctx, rows = self.build_context(entries)
            logits = self.model.forward(ctx, self.cache, rows)
        if commit:
            for e in entries:
                self.cache.commit(e.request, len(e.tokens))
        self.steps_run += 1
        if check:
            self.check_status()
        return logits

    def decode_graph(self, n: int):
        """The captured step for n single-token entries (None if n is beyond the buckets)."""
        from .decode_graph import DecodeGraph, bucket_for

        b = bucket_for(n)
        if b < 0 or b > self.cache.max_slots:
            b = self.cache.max_slots if n <= self.cache.max_slots else -1
        if b < 0:
            return None
        if b not in self._graphs:
            self._graphs[b] = DecodeGraph(self, [1] * b, [[0]] * b, padded=True)
        return self._graphs[b]

    MAX_SIGNATURE_GRAPHS = 48

    def graph_pool(self):
        """The memory pool that all captured steps of this runner share."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def _signature_graph(self, entries: Sequence[StepEntry]):
        """The captured step for this exact batch shape, once the shape has come before (None the first time)."""
        from .decode_graph import DecodeGraph

        sig = (tuple(len(e.tokens) for e in entries), tuple(tuple(e.want) for e in entries))
        graph = self._signature_graphs.get(sig)
        if graph is not None:
            self._signature_graphs[sig] = self._signature_graphs.pop(sig)         # most recently used last
            return graph
        self._signature_seen[sig] = self._signature_seen.get(sig, 0) + 1
        if self._signature_seen[sig] < 2 or sum(sig[0]) > 16384:
            return None
        if len(self._signature_graphs) >= self.MAX_SIGNATURE_GRAPHS:
            self._signature_graphs.pop(next(iter(self._signature_graphs)))        # the least recently used
            if len(self._signature_seen) > 4096:
                self._signature_seen.clear()
        graph = DecodeGraph(self, sig[0], sig[1], padded=False)
        self._signature_graphs[sig] = graph
        return graph

    def _reserve_for_step(self, entries: Sequence[StepEntry]) -> bool:
        """Pages for every entry's new tokens, or nothing at all (False)."""
        need: Dict[int, int] = {g.index: 0 for g in self.cache.groups}
        for e in entries:
            if not self.cache.can_reserve(e.request, len(e.tokens)):
                return False
            for gi, k in self.cache.pages_needed(e.request, len(e.tokens)).items():
                need[gi] += k
        if any(need[g.index] > g.pool.free_count for g in self.cache.groups):
            return False
        for e in entries:
            self.cache.reserve(e.request, len(e.tokens))
        return True

    def _run_captured(self, entries: Sequence[StepEntry]):
        """Steps whose shape has a captured graph go through it: (True, logits or None).  Anything
        else: (False, None), and the caller takes the general path."""
        no = (False, None)
        if len({e.request for e in entries}) != len(entries) or any(len(e.tokens) == 0 for e in entries):
            return no
        decode = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if decode and not all(self.cache.has_request(e.request) for e in entries):
            return no
        graph = self.decode_graph(len(entries)) if decode else None
        if graph is None:
            if any(w < 0 or w >= len(e.tokens) for e in entries for w in e.want):
                return no
            graph = self._signature_graph(entries)
        if graph is None:
            return no
        started = [e.request for e in entries if not self.cache.has_request(e.request)]
        if len(started) > self.cache.free_slot_count():
            return no
        for r in started:
            self.cache.begin_request(r)
        if not self._reserve_for_step(entries):
            for r in started:
                self.cache.end_request(r)
            return no                        # the general path raises the proper error
        tokens = [t for e in entries for t in e.tokens]
        logits = graph.replay([e.request for e in entries], tokens)
        self.graph_replays += 1
        if logits is None:
            return True, None
        return True, (logits[:len(entries)] if graph.padded else logits)

    def check_status(self) -> None:
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise StepError("a kernel reported: " + kernels.describe_status(word))

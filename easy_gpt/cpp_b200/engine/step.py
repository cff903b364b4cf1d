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

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import host, kernels
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
        self.last_graph = None             # the captured step that ran last (for accounting)

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
        n = len(entries)
        handles = np.fromiter((cache.handle(e.request, create=True) for e in entries), dtype=np.int64, count=n)
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=n)
        self._reserve(entries, handles, counts)
        T = int(counts.sum())
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        want_offsets = np.zeros(n + 1, dtype=np.int64)
        want_offsets[1:] = np.cumsum([len(e.want) for e in entries])
        R = int(want_offsets[n])
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int64, count=R)
        G = len(cache.groups)
        lib = cache._lib
        bound = int(lib.egh_step_bound(cache.core, n, T, R, kernels.QUERY_TILE))
        ring_index, host_buf, dev = self._buffers(bound)
        layout = np.zeros(2 * (9 + 2 * G), dtype=np.int64)
        widths = np.zeros(max(G, 1), dtype=np.int32)
        scalars = np.zeros(8, dtype=np.int64)
        rc = lib.egh_step_pack(cache.core, n, handles.ctypes.data, counts.ctypes.data, token_ids.ctypes.data,
                               want_offsets.ctypes.data, wants.ctypes.data, kernels.QUERY_TILE, kernels.SMALL_ENTRY_TOKENS,
                               host_buf.data_ptr(), host_buf.numel(), layout.ctypes.data, widths.ctypes.data, scalars.ctypes.data)
        if rc != 0:
            if token_ids.min() < -(1 << 31) or token_ids.max() >= (1 << 31):
                raise StepError("token ids do not fit 32 bits")
            raise StepError(f"packing the step failed with status {rc}")
        off = int(scalars[0])
        names = ["token_ids", "positions", "token_seq", "seq_starts", "seq_context", "seq_slots", "logit_rows",
                 "query_tiles", "small_tokens"]
        for g in cache.groups:
            names += [f"slot_map{g.index}", f"table{g.index}"]
        offsets = {name: (int(layout[2 * i]), int(layout[2 * i + 1])) for i, name in enumerate(names)}
        width = {g.index: int(widths[g.index]) for g in cache.groups}
        num_tiles, num_small = int(scalars[6]), int(scalars[7])
        hv = host_buf.numpy()

        def host_list(name):
            o, size = offsets[name]
            return hv[o:o + size].tolist()

        starts, context, slots = host_list("seq_starts"), host_list("seq_context"), host_list("seq_slots")
        dev[:off].copy_(host_buf[:off], non_blocking=True)
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
            host_seq_starts=starts, host_seq_context=context, host_seq_slots=slots,
            max_query_len=int(scalars[3]), max_context_len=int(scalars[4]),
            all_decode=bool(scalars[5]),
            query_tiles=view("query_tiles").view(num_tiles, 3) if num_tiles else None,
            small_tokens=view("small_tokens") if num_tiles and num_small else None,
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
            self.cache.zero_fresh_state()    # slots taken since the last step (by this step or by the scheduler)
            logits = self.model.forward(ctx, self.cache, rows)
        if commit:
            for e in entries:
                self.cache.commit(e.request, len(e.tokens))
        self.steps_run += 1
        if check:
            self.check_status()
        return logits

    def _handles(self, requests) -> np.ndarray:
        return np.fromiter((self.cache.handle(r, create=True) for r in requests), dtype=np.int64, count=len(requests))

    def _context_after(self, handles: np.ndarray, most_new_tokens: int) -> int:
        """Tokens the longest of these requests holds once the step's tokens are in (requests not yet live hold none)."""
        longest = int(self.cache._lib.egh_cache_max_length(self.cache.core, len(handles), handles.ctypes.data))
        return max(longest, 0) + most_new_tokens

    def decode_graph(self, n: int, context: int = 0):
        """The captured step for n single-token entries whose requests hold up to ``context`` tokens after it
        (0: as many as a request may hold); None if n is beyond the buckets."""
        from .decode_graph import DecodeGraph, bucket_for, context_pages

        b = bucket_for(n)
        if b < 0 or b > self.cache.max_slots:
            b = self.cache.max_slots if n <= self.cache.max_slots else -1
        if b < 0:
            return None
        most = self.cache.max_pages_per_request
        width = context_pages(context, self.cache.page_size, most) if context else most
        if (b, width) not in self._graphs:
            self._graphs[(b, width)] = DecodeGraph(self, [1] * b, [[0]] * b, padded=True, table_width=width)
        return self._graphs[(b, width)]

    def decode_graph_for(self, requests):
        """(graph, handles) for a decode step of these live requests."""
        handles = self._handles(requests)
        return self.decode_graph(len(requests), self._context_after(handles, 1)), handles

    MAX_SIGNATURE_GRAPHS = 48
    CAPTURE_MIXED_AFTER = 4            # times a shape of several entries is seen before it is captured

    def graph_pool(self):
        """The memory pool that all captured steps of this runner share."""
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def _signature_graph(self, entries: Sequence[StepEntry], handles: np.ndarray):
        """The captured step for this exact batch shape (and context bucket), once the shape has come before
        (None the first time)."""
        from .decode_graph import DecodeGraph, context_pages

        counts = tuple(len(e.tokens) for e in entries)
        width = context_pages(self._context_after(handles, max(counts)), self.cache.page_size, self.cache.max_pages_per_request)
        sig = (counts, tuple(tuple(e.want) for e in entries), width)
        graph = self._signature_graphs.get(sig)
        if graph is not None:
            self._signature_graphs[sig] = self._signature_graphs.pop(sig)         # most recently used last
            return graph
        self._signature_seen[sig] = self._signature_seen.get(sig, 0) + 1
        # A capture costs about as much as six eager steps.  One request's portions come again and again; a batch
        # of several requests rarely comes twice in the same shape (the number of decoding requests moves), so it
        # has to show that it does before it is captured.
        capture_after = 2 if len(sig[0]) == 1 else self.CAPTURE_MIXED_AFTER
        if self._signature_seen[sig] < capture_after or sum(sig[0]) > 16384:
            return None
        if len(self._signature_graphs) >= self.MAX_SIGNATURE_GRAPHS:
            self._signature_graphs.pop(next(iter(self._signature_graphs)))        # the least recently used
            if len(self._signature_seen) > 4096:
                self._signature_seen.clear()
        graph = DecodeGraph(self, sig[0], sig[1], padded=False, table_width=width)
        self._signature_graphs[sig] = graph
        return graph

    def _reserve(self, entries: Sequence[StepEntry], handles: np.ndarray, counts: np.ndarray) -> None:
        """Begins the step's new requests and takes the pages for every entry's tokens: all of it, or an
        exception with nothing changed."""
        from ..cache.manager import OutOfSlots
        from ..cache.page_pool import OutOfPages

        cache = self.cache
        info = np.zeros(3, dtype=np.int32)
        rc = cache._lib.egh_step_reserve(cache.core, len(entries), handles.ctypes.data, counts.ctypes.data, info.ctypes.data)
        if rc == 0:
            return
        for e in entries:                    # names that were made for requests which did not come to life
            if not cache.has_request(e.request):
                cache._forget(e.request, cache.handle(e.request))
        if rc == host.OUT_OF_PAGES:
            raise OutOfPages(f"group {info[0]}: the step needs {info[1]} new pages, {info[2]} are free")
        if rc == host.TOO_LONG:
            e = entries[int(info[0])]
            raise OutOfPages(f"request {e.request!r} would hold more tokens than a request may hold "
                             f"({cache.max_pages_per_request * cache.page_size})")
        if rc == host.OUT_OF_SLOTS:
            raise OutOfSlots(f"all {cache.max_slots} request slots are taken")
        raise StepError(f"reserving the step's pages failed with status {rc}")

    def _reserve_for_step(self, entries: Sequence[StepEntry]) -> bool:
        """Pages for every entry's new tokens (new requests are begun), or nothing at all (False)."""
        n = len(entries)
        handles = np.fromiter((self.cache.handle(e.request, create=True) for e in entries), dtype=np.int64, count=n)
        counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=n)
        try:
            self._reserve(entries, handles, counts)
        except Exception:
            return False
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
        if any(w < 0 or w >= len(e.tokens) for e in entries for w in e.want):
            return no
        handles = self._handles([e.request for e in entries])
        graph = self.decode_graph(len(entries), self._context_after(handles, 1)) if decode else None
        if graph is None:
            graph = self._signature_graph(entries, handles)
        if graph is None:
            self._forget_unborn(entries)
            return no
        if not self._reserve_for_step(entries):
            return no                        # the general path raises the proper error
        tokens = [t for e in entries for t in e.tokens]
        logits = graph.replay([e.request for e in entries], tokens, handles=handles)
        self.graph_replays += 1
        self.last_graph = graph
        if logits is None:
            return True, None
        return True, (logits[:len(entries)] if graph.padded else logits)

    def _forget_unborn(self, entries) -> None:
        """Names that were made for requests which have not come to life (the general path makes them again)."""
        for e in entries:
            if not self.cache.has_request(e.request):
                h = self.cache.handle(e.request)
                if h is not None:
                    self.cache._forget(e.request, h)

    def check_status(self) -> None:
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise StepError("a kernel reported: " + kernels.describe_status(word))

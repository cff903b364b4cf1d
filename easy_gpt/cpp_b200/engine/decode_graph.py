"""CUDA graphs for steps whose shape repeats.

A step is a fixed sequence of launches once it is known how many tokens every
entry brings and where logits are wanted (its *signature*); the only changing
inputs are small integer arrays (token ids, positions, cache positions, block
tables).  The sequence is captured once over static buffers; a step then costs
one host-to-device copy of the arrays and one graph launch instead of a few
hundred launches.  Decode steps (every entry brings one token) are captured per
batch-size bucket and padded; other signatures (a prompt portion of the chunk
size, say) are captured when they come a second time (batches of several entries: a fourth time).  (The reference captures a graph only for the attention of
one layer at batch 1 and re-captures whenever a pointer changes,
src/cuda/ops/self_attn.cu:750-828.)

Rows that pad a batch up to its bucket are given position 0, the group's
scratch page and the scratch state slot (one past the last slot a request can
hold), so they read and write nothing that belongs to a request.
"""
from __future__ import annotations

import gc
from typing import List, Sequence

import numpy as np
import torch

from .. import host, kernels
from ..parts.base import GroupTables, StepContext

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
MIN_CONTEXT_BUCKET = 512           # tokens: shorter contexts share the smallest captured step


def context_pages(tokens: int, page_size: int, most: int) -> int:
    """Block-table width (pages) of the captured step that serves requests of up to ``tokens`` tokens:
    the next power of two of tokens, at least MIN_CONTEXT_BUCKET, at most what a request may hold.
    A request outgrows its bucket log2(length) times in its life, and each bucket's step is planned
    for the contexts it really sees, not for the longest a request may ever get."""
    bucket = MIN_CONTEXT_BUCKET
    while bucket < tokens:
        bucket *= 2
    return max(1, min(most, -(-bucket // page_size)))


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return -1


class DecodeGraph:
    """A captured step for one batch *signature*: how many tokens each entry brings and where logits
    are wanted.  ``padded`` (decode buckets): fewer entries than the signature's may be replayed; the
    rest are padding rows."""

    def __init__(self, runner, counts: Sequence[int], wants: Sequence[Sequence[int]], padded: bool, table_width: int = 0):
        """``table_width``: pages per block-table row that the captured step carries (0: as many as a request
        may hold).  The step serves requests of up to table_width * page_size tokens; its launch plans
        (how many CTAs share a request's keys) are made for that context length."""
        self.runner = runner
        self.counts = [int(c) for c in counts]
        self.padded = padded
        self.bucket = n = len(self.counts)
        self.tokens = T = sum(self.counts)
        self.all_decode = all(c == 1 for c in self.counts)
        cache = runner.cache
        dev = runner.device
        self.table_width = W = min(table_width, cache.max_pages_per_request) if table_width else cache.max_pages_per_request
        self.widths = {g.index: W for g in cache.groups}
        layout = [("token_ids", T), ("positions", T), ("seq_context", n), ("seq_slots", n)]
        for g in cache.groups:
            layout += [(f"slot_map{g.index}", T), (f"table{g.index}", n * self.widths[g.index])]
        self.offsets, off = {}, 0
        for name, size in layout:
            self.offsets[name] = (off, size)
            off += (size + 3) & ~3
        self.size = off
        self.meta = torch.zeros(off, dtype=torch.int32, device=dev)
        self.staging = [torch.zeros(off, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.staging_events: List = [None] * 4
        self.next_staging = 0
        # what depends on the signature alone
        starts = np.zeros(n + 1, dtype=np.int32)
        starts[1:] = np.cumsum(self.counts)
        self.starts = starts
        self._counts32 = np.asarray(self.counts, dtype=np.int32)
        self._off_slot_map = np.asarray([self.offsets[f"slot_map{g.index}"][0] for g in cache.groups] or [0], dtype=np.int64)
        self._off_table = np.asarray([self.offsets[f"table{g.index}"][0] for g in cache.groups] or [0], dtype=np.int64)
        token_seq = np.repeat(np.arange(n, dtype=np.int32), self.counts)
        rows = [int(starts[i]) + int(w) for i, ws in enumerate(wants) for w in ws]
        tiles, small = kernels.query_tiles_of(starts, self.counts)
        to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)

        def view(name):
            o, size = self.offsets[name]
            return self.meta[o:o + size]

        self.ctx = StepContext(
            dtype=runner.model.dtype, device=dev, num_tokens=T, num_seqs=n,
            token_ids=view("token_ids"), positions=view("positions"), token_seq=to_dev(token_seq),
            seq_starts=to_dev(starts), seq_context=view("seq_context"), seq_slots=view("seq_slots"), status=runner.status,
            groups={g.index: GroupTables(g.page_size, view(f"table{g.index}").view(n, self.widths[g.index]),
                                         view(f"slot_map{g.index}")) for g in cache.groups},
            host_seq_starts=starts.tolist(), host_seq_context=[0] * n, host_seq_slots=[0] * n,
            max_query_len=max(self.counts), max_context_len=W * cache.page_size,
            all_decode=self.all_decode,
            query_tiles=to_dev(np.asarray(tiles, dtype=np.int32).reshape(-1, 3)) if tiles else None,
            small_tokens=to_dev(np.asarray(small, dtype=np.int32)) if tiles and small else None)
        self.rows = to_dev(np.asarray(rows, dtype=np.int32)) if rows else None
        self.all_rows = rows == list(range(T))
        self._fill_padding(self.staging[0].numpy(), 0)
        self.meta.copy_(self.staging[0])
        # run once eagerly (library handles and workspaces come into being), then capture
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            runner.model.forward(self.ctx, cache, self.rows, all_rows=self.all_rows)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        before = kernels.launch_count
        self.graph = torch.cuda.CUDAGraph()
        # Captured by hand rather than with torch.cuda.graph(): that context collects garbage and empties the
        # allocator's cache on entry, tens of milliseconds per capture, and every eager step after it pays for
        # fresh device allocations.  No garbage collection while the stream is capturing either: freeing an older
        # graph or tensor there is a CUDA call that is not allowed during a capture and would invalidate it.
        # All captured steps of a runner share one memory pool: they never run at the same time.
        was_enabled = gc.isenabled()
        gc.disable()
        capture_stream = torch.cuda.Stream(device=dev)
        capture_stream.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(capture_stream):
                self.graph.capture_begin(pool=runner.graph_pool())
                try:
                    self.logits = runner.model.forward(self.ctx, cache, self.rows, all_rows=self.all_rows)
                finally:
                    self.graph.capture_end()
        finally:
            if was_enabled:
                gc.enable()
        torch.cuda.current_stream().wait_stream(capture_stream)
        self.launches = kernels.launch_count - before      # our own kernels inside one replay

    def _fill_padding(self, hv: np.ndarray, start_row: int) -> None:
        """Rows from ``start_row`` on are padding (every entry of a padded signature brings one token)."""
        cache = self.runner.cache
        B = self.bucket
        first_token = int(self.starts[start_row])
        for name, first in (("token_ids", first_token), ("positions", first_token), ("seq_context", start_row)):
            o, size = self.offsets[name]
            hv[o + first:o + size] = 0
        o, size = self.offsets["seq_slots"]
        hv[o + start_row:o + size] = cache.max_slots           # the scratch slot: no request's state
        for g in cache.groups:
            o, size = self.offsets[f"slot_map{g.index}"]
            hv[o + first_token:o + size] = g.scratch_page * g.page_size
            o, _ = self.offsets[f"table{g.index}"]
            W = self.widths[g.index]
            hv[o + start_row * W:o + B * W] = g.scratch_page

    def replay(self, requests: Sequence, tokens, tokens_on_device: bool = False, handles=None) -> torch.Tensor:
        """requests: ids of the live requests of this step, in the signature's order (fewer than the
        signature's only if it is padded); pages for their new tokens are already reserved.  tokens:
        their token ids, flat, in order (ignored with tokens_on_device: the device already holds them).
        Returns the static logits buffer; rows of padding entries are to be ignored."""
        cache = self.runner.cache
        n = len(requests)
        assert n == self.bucket or self.padded
        i = self.next_staging
        self.next_staging = (i + 1) % len(self.staging)
        if self.staging_events[i] is not None:
            self.staging_events[i].synchronize()
        hv = self.staging[i].numpy()
        if not tokens_on_device:
            o, _ = self.offsets["token_ids"]
            hv[o:o + int(self.starts[n])] = np.asarray(tokens, dtype=np.int32)
        # (with tokens_on_device the ids were put there by set_tokens_from_device; the rows that pad the
        # bucket keep whatever id they had: any valid id will do for them)
        # positions, cached lengths, slots, cache positions and block-table rows: packed by the host runtime
        if handles is None:
            handles = np.fromiter((cache.handle(r) for r in requests), dtype=np.int64, count=n)
        rc = cache._lib.egh_replay_pack(cache.core, n, handles.ctypes.data, self._counts32.ctypes.data, self.staging[i].data_ptr(),
                                        self.offsets["positions"][0], self.offsets["seq_context"][0], self.offsets["seq_slots"][0],
                                        self._off_slot_map.ctypes.data, self._off_table.ctypes.data, self.table_width)
        if rc != 0:
            raise RuntimeError("a token of a captured step has no cache page" if rc == host.NO_PAGE
                               else f"packing a captured step failed with status {rc}")
        if n < self.bucket:
            self._fill_padding(hv, n)
        if tokens_on_device:
            # token ids stay as the device left them (the sampler's output was copied in)
            o, size = self.offsets["token_ids"]
            first = o + size
            self.meta[first:].copy_(self.staging[i][first:], non_blocking=True)
        else:
            self.meta.copy_(self.staging[i], non_blocking=True)
        if self.staging_events[i] is None:
            self.staging_events[i] = torch.cuda.Event()
        self.staging_events[i].record()
        cache.zero_fresh_state()             # slots taken since the last step start from zeroed state
        self.graph.replay()
        return self.logits

    def set_tokens_from_device(self, tokens: torch.Tensor) -> None:
        o, _ = self.offsets["token_ids"]
        self.meta[o:o + tokens.numel()].copy_(tokens, non_blocking=True)

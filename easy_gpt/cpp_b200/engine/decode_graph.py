"""CUDA graphs for steps in which every request brings exactly one token.

Such a step is a fixed sequence of launches whose only changing inputs are small
integer arrays (token ids, positions, cache positions, block tables).  For each
batch-size bucket the sequence is captured once over static buffers; a step then
costs one host-to-device copy of the arrays and one graph launch instead of a
few hundred launches.  (The reference captures a graph only for the attention of
one layer at batch 1 and re-captures whenever a pointer changes,
src/cuda/ops/self_attn.cu:750-828.)

Rows that pad a batch up to its bucket are given position 0 and the group's
scratch page, so they read and write nothing that belongs to a request.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..parts.base import GroupTables, StepContext

BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return -1


class DecodeGraph:
    def __init__(self, runner, bucket: int):
        self.runner = runner
        self.bucket = B = bucket
        cache = runner.cache
        dev = runner.device
        self.widths = {g.index: cache.max_pages_per_request for g in cache.groups}
        layout = [("token_ids", B), ("positions", B), ("seq_context", B), ("seq_slots", B)]
        for g in cache.groups:
            layout += [(f"slot_map{g.index}", B), (f"table{g.index}", B * self.widths[g.index])]
        self.offsets, off = {}, 0
        for name, size in layout:
            self.offsets[name] = (off, size)
            off += (size + 3) & ~3
        self.size = off
        self.meta = torch.zeros(off, dtype=torch.int32, device=dev)
        self.staging = [torch.zeros(off, dtype=torch.int32).pin_memory() for _ in range(4)]
        self.staging_events: List = [None] * 4
        self.next_staging = 0
        arange = torch.arange(B + 1, dtype=torch.int32, device=dev)

        def view(name):
            o, size = self.offsets[name]
            return self.meta[o:o + size]

        self.ctx = StepContext(
            dtype=runner.model.dtype, device=dev, num_tokens=B, num_seqs=B,
            token_ids=view("token_ids"), positions=view("positions"), token_seq=arange[:B].clone(),
            seq_starts=arange, seq_context=view("seq_context"), seq_slots=view("seq_slots"), status=runner.status,
            groups={g.index: GroupTables(g.page_size, view(f"table{g.index}").view(B, self.widths[g.index]),
                                         view(f"slot_map{g.index}")) for g in cache.groups},
            host_seq_starts=list(range(B + 1)), host_seq_context=[0] * B, host_seq_slots=[0] * B,
            max_query_len=1, max_context_len=cache.max_pages_per_request * cache.page_size, all_decode=True)
        self.rows = arange[:B].clone()
        self._fill_padding(self.staging[0].numpy(), 0)
        self.meta.copy_(self.staging[0])
        # run once eagerly (library handles and workspaces come into being), then capture
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            runner.model.forward(self.ctx, cache, self.rows, all_rows=True)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        from .. import kernels
        before = kernels.launch_count
        self.graph = torch.cuda.CUDAGraph()
        # No garbage collection while the stream is capturing: freeing an older engine's graphs or
        # tensors there is a CUDA call that is not allowed during a capture and would invalidate it.
        gc.collect()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = runner.model.forward(self.ctx, cache, self.rows, all_rows=True)
        finally:
            if was_enabled:
                gc.enable()
        self.launches = kernels.launch_count - before      # our own kernels inside one replay

    def _fill_padding(self, hv: np.ndarray, start_row: int) -> None:
        cache = self.runner.cache
        B = self.bucket
        for name in ("token_ids", "positions", "seq_context", "seq_slots"):
            o, _ = self.offsets[name]
            hv[o + start_row:o + B] = 0
        for g in cache.groups:
            o, _ = self.offsets[f"slot_map{g.index}"]
            hv[o + start_row:o + B] = g.scratch_page * g.page_size
            o, _ = self.offsets[f"table{g.index}"]
            W = self.widths[g.index]
            hv[o + start_row * W:o + B * W] = g.scratch_page

    def replay(self, requests: Sequence, tokens: Sequence[int], tokens_on_device: bool = False) -> torch.Tensor:
        """requests: ids of the n <= bucket live requests, each advancing by one token
        (pages already reserved).  Returns the static logits buffer [bucket, vocab];
        rows beyond n are padding."""
        cache = self.runner.cache
        n = len(requests)
        i = self.next_staging
        self.next_staging = (i + 1) % len(self.staging)
        if self.staging_events[i] is not None:
            self.staging_events[i].synchronize()
        hv = self.staging[i].numpy()
        lengths = np.fromiter((cache.length_of(r) for r in requests), dtype=np.int32, count=n)
        slots = np.fromiter((cache.slot_of(r) for r in requests), dtype=np.int32, count=n)

        def put(name, arr):
            o, _ = self.offsets[name]
            hv[o:o + len(arr)] = arr

        if not tokens_on_device:
            put("token_ids", np.asarray(tokens, dtype=np.int32))
        # (with tokens_on_device the ids were put there by set_tokens_from_device; the rows that pad the
        # bucket keep whatever id they had: any valid id will do for them)
        put("positions", lengths)
        put("seq_context", lengths)
        put("seq_slots", slots)
        for g in cache.groups:
            W = self.widths[g.index]
            rows = g.tables[slots]                                           # [n, W]
            pages = rows[np.arange(n), lengths // g.page_size].astype(np.int64)
            put(f"slot_map{g.index}", (pages * g.page_size + lengths % g.page_size).astype(np.int32))
            o, _ = self.offsets[f"table{g.index}"]
            hv[o:o + n * W] = rows.reshape(-1)
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
        self.graph.replay()
        return self.logits

    def set_tokens_from_device(self, tokens: torch.Tensor) -> None:
        o, _ = self.offsets["token_ids"]
        self.meta[o:o + tokens.numel()].copy_(tokens, non_blocking=True)

"""Sampling of next tokens from float32 logits on the device: one kernel launch
for the whole batch, greedy rows and sampled rows together."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams
from .rng import uniform


class Sampler:
    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self._cap:
            return
        self._cap = max(rows, 2 * self._cap)
        # pinned float32 blocks [4, cap]: temperature, top_p, uniform, top_k (as int bits).  Several in turn, each
        # with the event of the copy that last read it: the host runs ahead of the device, and a block written
        # again before its copy has run would hand that step the next step's numbers.
        self._hosts = [torch.empty((4, self._cap), dtype=torch.float32).pin_memory() for _ in range(4)]
        self._host_events = [None] * len(self._hosts)
        self._host_turn = 0
        self._dev = torch.empty((4, self._cap), dtype=torch.float32, device=self.device)
        # two output buffers in turn: a step's tokens stay readable (they feed the next step on the
        # device, and their copy to the host is read late) while the next step's are being written
        self._outs = [torch.empty(self._cap, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._out_hosts = [torch.empty(self._cap, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._turn = 0
        self._out = self._outs[0]
        self._out_host = self._out_hosts[0]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], request_ids: Sequence[int],
               token_indices: Sequence[int]) -> torch.Tensor:
        """Returns int32 tokens [rows] on the device.  Row r is sampled with
        params[r]; its uniform number is keyed by (seed, request_ids[r], token_indices[r])."""
        rows = logits.shape[0]
        assert len(params) == len(request_ids) == len(token_indices) == rows
        self._grow(rows)
        self._turn ^= 1
        self._out, self._out_host = self._outs[self._turn], self._out_hosts[self._turn]
        if all(p.is_greedy for p in params):
            kernels.argmax(logits, self._out)
            return self._out[:rows]
        i = self._host_turn
        self._host_turn = (i + 1) % len(self._hosts)
        if self._host_events[i] is not None:
            self._host_events[i].synchronize()
        host = self._hosts[i]
        h = host.numpy()
        for r, p in enumerate(params):
            h[0, r] = 0.0 if p.is_greedy else p.temperature
            h[1, r] = p.top_p
            h[2, r] = 0.0 if p.is_greedy else uniform(p.seed, int(request_ids[r]), int(token_indices[r]))
        h[3, :rows].view(np.int32)[:] = [p.top_k for p in params]
        self._dev[:, :rows].copy_(host[:, :rows], non_blocking=True)
        if self._host_events[i] is None:
            self._host_events[i] = torch.cuda.Event()
        self._host_events[i].record()
        kernels.sample(logits, self._dev[0], self._dev[3].view(torch.int32), self._dev[1], self._dev[2], self._out)
        return self._out[:rows]

    def to_host_async(self, tokens: torch.Tensor):
        """Starts the copy of ``tokens`` (the result of the last ``sample``) to pinned host memory and
        returns a function that waits for it and gives the Python ints."""
        n = tokens.numel()
        host = self._out_host
        host[:n].copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()

        def result():
            event.synchronize()
            return host[:n].tolist()

        return result

    def to_host(self, tokens: torch.Tensor) -> list:
        """Device tokens -> Python ints (synchronises the stream)."""
        n = tokens.numel()
        self._out_host[:n].copy_(tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:n].tolist()

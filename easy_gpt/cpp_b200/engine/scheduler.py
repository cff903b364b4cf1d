"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.  Host code over the cache manager's
bookkeeping; it never touches the device, so its decisions are tested without
one.  The decisions are made in C++ (``csrc/host/scheduler_core.hpp``), which
knows requests by their lengths; this module is its face in Python and keeps
what the decisions do not need: token ids and sampling parameters.

It follows the rounds of the reference's ContinuousBatchServer
(src/continuous_batch_server.cpp:71-86): a FIFO of waiting requests, at most
``prefill_batch`` admissions per round and at most ``max_active`` live requests
(:88-101), every decoding request advances by one token per round (:160-200), a
request ends on EOS — which is emitted — or at its length limit (:141-149,
189-197), and its slot and cache are given back at once (:222-260).  What the
reference does not have: one mixed step instead of separate prefill and decode
rounds, a token budget with portions of prompts, and pages that can run out.

When pages run out
  * at admission, the request waits (FIFO order is kept: nothing overtakes it);
  * for a request already running, the most recently admitted running request is
    preempted: everything it holds is given back and it returns to the FRONT of
    the waiting queue with the tokens it has generated; later it is prefilled
    again over prompt + generated tokens and continues.  Its outputs are the
    same as without preemption (sampling numbers are keyed by request and token
    index);
  * a request that cannot fit even alone in an empty pool fails with an error.
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional, Sequence

import numpy as np

from .. import host
from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class SchedulerOptions:
    max_batch_tokens: int = 2048       # tokens per step
    chunk_size: int = 512              # longest portion of a prompt in one step
    max_active: int = 16               # live requests (src/cli_options.cpp: --serve-max-active)
    prefill_batch: int = 4             # admissions per step (--serve-prefill-batch)
    eos_token_id: int = -1             # < 0: no EOS
    max_positions: int = 1 << 30       # max_position_embeddings


_STATES = ("waiting", "running", "finished")
_REASONS = (None, "empty", "eos", "length", "max_positions", "error")
# fields of egh_sched_request
_PROMPT_LEN, _OUTPUT_LEN, _MAX_NEW, _COMPUTED, _STATE, _REASON, _ERROR, _PENDING, _PREEMPTIONS, _ADMITTED_AT = range(10)


class Request:
    """A request as its owner sees it: token ids, sampling parameters and the output so far are kept here;
    how far it has come (``computed``, ``state``, ``pending``, ...) is read from the scheduler."""

    def __init__(self, scheduler: "Scheduler", rid: int, prompt: List[int], params: SamplingParams, max_new_tokens: int):
        self._scheduler = scheduler
        self.id = rid
        self.prompt = prompt
        self.params = params
        self.max_new_tokens = max_new_tokens
        self.output: List[int] = []

    def _field(self, index: int) -> int:
        return self._scheduler._request_fields(self.id)[index]

    @property
    def computed(self) -> int:
        """Tokens whose keys/values are in the cache."""
        return self._field(_COMPUTED)

    @property
    def state(self) -> str:
        """waiting | running | finished"""
        return _STATES[self._field(_STATE)]

    @property
    def finish_reason(self) -> Optional[str]:
        return _REASONS[self._field(_REASON)]

    @property
    def error(self) -> Optional[str]:
        return self._scheduler._error_text(self, self._field(_ERROR))

    @property
    def preemptions(self) -> int:
        return self._field(_PREEMPTIONS)

    @property
    def admitted_at(self) -> int:
        """Admission counter, for "most recently admitted"."""
        return self._field(_ADMITTED_AT)

    @property
    def pending(self) -> int:
        """Tokens sampled on the device whose ids the host has not read yet (0 or 1 between steps)."""
        return self._field(_PENDING)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def known(self) -> int:
        """Tokens that exist for this request, the one still on its way from the device included."""
        return len(self.prompt) + len(self.output) + self.pending

    def token_slice(self, start: int, count: int) -> List[int]:
        """tokens[start : start + count] without building the whole list (a decode step asks for one token).
        A token whose id is still pending cannot be given (the caller feeds it on the device)."""
        n = len(self.prompt)
        if start + count > n + len(self.output):
            raise ValueError(f"request {self.id}: token {start + count - 1} is still on the device")
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    def __repr__(self):
        return f"Request(id={self.id}, prompt={len(self.prompt)} tokens, output={len(self.output)} tokens, state={self.state})"


@dataclass
class Scheduled:
    request: Request
    start: int                         # first position fed this step
    count: int                         # tokens fed
    samples: bool                      # the portion reaches the last known token: its logits give the next token
    pending: int = 0                   # the request's tokens still on the device when the step was scheduled (0 or 1)


@dataclass
class SchedulerStats:
    steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    failed: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, options: SchedulerOptions):
        if options.max_batch_tokens <= 0 or options.chunk_size <= 0 or options.max_active <= 0 or options.prefill_batch <= 0:
            raise ValueError("scheduler limits must be positive")
        self.cache = cache
        self.opt = options
        self._lib = host.library()
        self._core = self._lib.egh_sched_create(cache.core, options.max_batch_tokens, options.chunk_size, options.max_active,
                                                options.prefill_batch, options.eos_token_id, options.max_positions)
        if not self._core:
            raise ValueError("the scheduler could not be made from these options")
        self._requests: Dict[int, Request] = {}
        self._fields = (ctypes.c_longlong * 10)()
        self._batch_cap = max(options.max_active, cache.max_slots) + 1
        self._batch = np.zeros(5 * self._batch_cap, dtype=np.int64)

    def __del__(self):
        core = getattr(self, "_core", None)
        if core:
            self._core = None
            self._lib.egh_sched_destroy(core)

    # -- what the C++ side knows ---------------------------------------------------
    def _request_fields(self, rid: int):
        if self._lib.egh_sched_request(self._core, rid, self._fields) != host.OK:
            raise KeyError(rid)
        return self._fields

    def _error_text(self, req: Request, code: int) -> Optional[str]:
        if code == 0:
            return None
        if code == 1:
            return (f"prompt of {len(req.prompt)} tokens leaves no room under "
                    f"max_position_embeddings={self.opt.max_positions}")
        if code == 2:
            return f"prompt of {len(req.prompt)} tokens cannot fit the cache even alone"
        return "the cache cannot hold this request even alone"

    def _listed(self, which: int) -> List[Request]:
        cap = len(self._requests) + 1
        ids = (ctypes.c_longlong * cap)()
        n = self._lib.egh_sched_list(self._core, which, ids, cap)
        return [self._requests[i] for i in ids[:n]]

    @property
    def waiting(self) -> Deque[Request]:
        return deque(self._listed(0))

    @property
    def running(self) -> List[Request]:
        return self._listed(1)

    @property
    def finished(self) -> List[Request]:
        return self._listed(2)

    @property
    def stats(self) -> SchedulerStats:
        out = (ctypes.c_longlong * 6)()
        self._lib.egh_sched_stats(self._core, out)
        return SchedulerStats(*[int(v) for v in out])

    # -- intake ---------------------------------------------------------------
    def add(self, prompt: Sequence[int], params: SamplingParams, max_new_tokens: int) -> Request:
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        prompt = list(prompt)
        # an empty prompt is answered at once (src/continuous_batch_server.cpp:285-291)
        rid = int(self._lib.egh_sched_add(self._core, len(prompt), int(max_new_tokens)))
        req = Request(self, rid, prompt, params, max_new_tokens)
        self._requests[rid] = req
        return req

    def forget(self, req: Request) -> None:
        """Drops the record of a finished request (a long-running caller that has read its output)."""
        if req.state == "finished":
            self._lib.egh_sched_forget(self._core, req.id)
            self._requests.pop(req.id, None)

    def has_work(self) -> bool:
        return bool(self._lib.egh_sched_has_work(self._core))

    # -- one round -----------------------------------------------------------------
    def schedule(self) -> List[Scheduled]:
        """Decides the next step's batch and reserves its cache pages."""
        n = self._lib.egh_sched_schedule(self._core, self._batch.ctypes.data, self._batch_cap)
        if n < 0:
            raise RuntimeError(f"the scheduler failed with status {n}")
        flat = self._batch[:5 * n].tolist()
        requests = self._requests
        return [Scheduled(requests[flat[i]], flat[i + 1], flat[i + 2], bool(flat[i + 3]), flat[i + 4]) for i in range(0, 5 * n, 5)]

    def update(self, batch: Sequence[Scheduled], next_tokens: Sequence[int]) -> List[Request]:
        """After the step ran: ``next_tokens`` holds one sampled token for every
        entry with ``samples`` (in batch order).  Returns the requests that finished."""
        self.launched(batch)
        return self.resolve(batch, next_tokens)

    @staticmethod
    def _flat(batch: Sequence[Scheduled]) -> np.ndarray:
        return np.array([v for s in batch for v in (s.request.id, s.start, s.count, int(s.samples))], dtype=np.int64)

    def launched(self, batch: Sequence[Scheduled]) -> None:
        """The step has been handed to the device: its tokens count as cached, and every sampling
        entry has one token on its way (``pending``) whose id ``resolve`` will bring."""
        flat = self._flat(batch)
        rc = self._lib.egh_sched_launched(self._core, flat.ctypes.data, len(batch))
        if rc == host.EXCEEDS_RESERVED:
            raise ValueError("a launched entry exceeds what was reserved for its request")
        if rc != host.OK:
            raise RuntimeError(f"the scheduler failed with status {rc}")

    def resolve(self, batch: Sequence[Scheduled], next_tokens: Sequence[int]) -> List[Request]:
        """The sampled tokens of a launched step have reached the host.  A request that had ended
        meanwhile (its previous token was EOS while this step was already on the device) drops its token."""
        sampling = [s for s in batch if s.samples]
        tokens = np.array([int(t) for t in next_tokens], dtype=np.int64)
        if len(tokens) < len(sampling):
            raise ValueError("fewer tokens than sampling entries")
        flat = self._flat(batch)
        actions = np.zeros(max(len(sampling), 1), dtype=np.int32)
        rc = self._lib.egh_sched_resolve(self._core, flat.ctypes.data, len(batch), tokens.ctypes.data, actions.ctypes.data)
        if rc < 0:
            raise RuntimeError(f"the scheduler failed with status {rc}")
        done = []
        for s, token, action in zip(sampling, tokens.tolist(), actions.tolist()):
            if action == 0:
                continue
            s.request.output.append(token)
            if action == 2:
                done.append(s.request)
        return done

    def advance_decoded(self, req: Request, tokens: Sequence[int]) -> None:
        """Tokens decoded outside the scheduler (a benchmark loop that feeds the device itself): they join the
        output, and all but the last count as cached, which the caller has committed to the cache manager."""
        rc = self._lib.egh_sched_advance(self._core, req.id, len(tokens))
        if rc != host.OK:
            raise ValueError(f"request {req.id} cannot be advanced by {len(tokens)} tokens")
        req.output += [int(t) for t in tokens]

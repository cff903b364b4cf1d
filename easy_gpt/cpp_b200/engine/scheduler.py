"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.  Pure host code over the cache manager's
bookkeeping; it never touches the device, so its decisions are tested without
one.

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

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

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


@dataclass(eq=False)
class Request:
    id: int
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    output: List[int] = field(default_factory=list)
    computed: int = 0                  # tokens whose keys/values are in the cache
    state: str = "waiting"             # waiting | running | finished
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1              # admission counter, for "most recently admitted"
    pending: int = 0                   # tokens sampled on the device whose ids the host has not read yet (0 or 1)

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


@dataclass
class Scheduled:
    request: Request
    start: int                         # first position fed this step
    count: int                         # tokens fed
    samples: bool                      # the portion reaches the last known token: its logits give the next token


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
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.stats = SchedulerStats()
        self._admissions = 0
        self._next_id = 0

    # -- intake ---------------------------------------------------------------
    def add(self, prompt: Sequence[int], params: SamplingParams, max_new_tokens: int) -> Request:
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        req = Request(self._next_id, list(prompt), params, max_new_tokens)
        self._next_id += 1
        if not req.prompt:
            # the reference answers an empty prompt at once (src/continuous_batch_server.cpp:285-291)
            self._finish(req, "empty")
            return req
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- helpers ------------------------------------------------------------------
    def _pool_tokens(self) -> int:
        return min(g.pool.num_pages for g in self.cache.groups) * self.cache.page_size if self.cache.groups else 1 << 60

    def _finish(self, req: Request, reason: str, error: Optional[str] = None) -> None:
        if self.cache.has_request(req.id):
            self.cache.end_request(req.id)
        if req.state == "running":
            self.running.remove(req)
        elif req.state == "waiting" and req in self.waiting:
            self.waiting.remove(req)
        req.state, req.finish_reason, req.error = "finished", reason, error
        self.finished.append(req)
        if error:
            self.stats.failed += 1
        else:
            self.stats.finished += 1

    def _preempt(self, victim: Request) -> None:
        self.cache.end_request(victim.id)
        self.running.remove(victim)
        victim.computed = 0
        victim.state = "waiting"
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(victim)

    def _limit_error(self, req: Request) -> Optional[str]:
        total = len(req.prompt) + 1
        if total > self.opt.max_positions:
            return f"prompt of {len(req.prompt)} tokens leaves no room under max_position_embeddings={self.opt.max_positions}"
        if total > self._pool_tokens() or total > self.cache.max_pages_per_request * self.cache.page_size:
            return f"prompt of {len(req.prompt)} tokens cannot fit the cache even alone"
        return None

    # -- one round -----------------------------------------------------------------
    def schedule(self) -> List[Scheduled]:
        """Decides the next step's batch and reserves its cache pages."""
        budget = self.opt.max_batch_tokens
        batch: List[Scheduled] = []

        # 1. every request that has all its known tokens but one in the cache decodes one token
        for req in list(self.running):
            if req.state != "running" or req.known - req.computed != 1 or budget <= 0:
                continue
            if req.pending and (len(req.output) + req.pending >= req.max_new_tokens or req.known >= self.opt.max_positions):
                continue                       # its pending token is its last one: it ends when the token is read
            while not self.cache.can_reserve(req.id, 1):
                victim = max(self.running, key=lambda r: r.admitted_at)
                scheduled_victim = next((s for s in batch if s.request is victim), None)
                if scheduled_victim is not None:
                    batch.remove(scheduled_victim)
                    budget += scheduled_victim.count
                only_one = len(self.running) == 1
                self._preempt(victim)
                if victim is req:
                    if only_one:
                        # alone and still too large: it can never go on
                        self.waiting.popleft()
                        self._finish(req, "error", "the cache cannot hold this request even alone")
                    break
            if req.state != "running":
                continue
            self.cache.reserve(req.id, 1)
            batch.append(Scheduled(req, req.computed, 1, True))
            budget -= 1

        # 2. requests in the middle of their prompt (or being recomputed) get their next portion
        for req in self.running:
            left = req.known - req.computed
            if left <= 1 or budget <= 0 or req.pending:
                continue                       # (a portion needs all its token ids on the host)
            n = min(left, self.opt.chunk_size, budget)
            if not self.cache.can_reserve(req.id, n):
                continue                       # waits for pages; decoding requests will free some or be preempted
            self.cache.reserve(req.id, n)
            batch.append(Scheduled(req, req.computed, n, req.computed + n == req.known))
            budget -= n

        # 3. admissions, FIFO, while slots, pages and budget last
        admitted = 0
        while (self.waiting and admitted < self.opt.prefill_batch and len(self.running) < self.opt.max_active
               and budget > 0 and self.cache.free_slot_count() > 0):
            req = self.waiting[0]
            if req.pending:
                break                          # preempted while its last token was on its way: wait for it
            err = self._limit_error(req)
            if err:
                self.waiting.popleft()
                self._finish(req, "error", err)
                continue
            n = min(req.known, self.opt.chunk_size, budget)
            # keep one page per running request in reserve, so that admissions do not starve decoding
            self.cache.begin_request(req.id)
            if not self.cache.can_reserve(req.id, n, spare=len(self.running)):
                self.cache.end_request(req.id)
                break
            self.cache.reserve(req.id, n)
            self.waiting.popleft()
            req.state = "running"
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)
            batch.append(Scheduled(req, 0, n, n == req.known))
            budget -= n
            admitted += 1

        if not batch and any(r.pending for r in self.running):
            return batch                       # everything live waits for a token that is on its way
        if not batch and self.running:
            # nothing fits although requests are live (all stuck in their prompts): make room
            victim = max(self.running, key=lambda r: r.admitted_at)
            if len(self.running) == 1:
                self._finish(victim, "error", "the cache cannot hold this request even alone")
            else:
                self._preempt(victim)
            return self.schedule()
        if batch:
            self.stats.steps += 1
        return batch

    def update(self, batch: Sequence[Scheduled], next_tokens: Sequence[int]) -> List[Request]:
        """After the step ran: ``next_tokens`` holds one sampled token for every
        entry with ``samples`` (in batch order).  Returns the requests that finished."""
        self.launched(batch)
        return self.resolve(batch, next_tokens)

    def launched(self, batch: Sequence[Scheduled]) -> None:
        """The step has been handed to the device: its tokens count as cached, and every sampling
        entry has one token on its way (``pending``) whose id ``resolve`` will bring."""
        for s in batch:
            req = s.request
            self.cache.commit(req.id, s.count)
            req.computed += s.count
            if s.count == 1 and s.start >= len(req.prompt):
                self.stats.decode_tokens += 1
            else:
                self.stats.prompt_tokens += s.count
            if s.samples:
                req.pending += 1

    def resolve(self, batch: Sequence[Scheduled], next_tokens: Sequence[int]) -> List[Request]:
        """The sampled tokens of a launched step have reached the host.  A request that had ended
        meanwhile (its previous token was EOS while this step was already on the device) drops its token."""
        done = []
        it = iter(next_tokens)
        for s in batch:
            if not s.samples:
                continue
            req = s.request
            token = int(next(it))
            if req.state == "finished":
                continue
            req.pending -= 1
            req.output.append(token)
            reason = None
            if self.opt.eos_token_id >= 0 and token == self.opt.eos_token_id:
                reason = "eos"                                  # the EOS token itself is emitted
            elif len(req.output) >= req.max_new_tokens:
                reason = "length"
            elif req.known + 1 > self.opt.max_positions:
                reason = "max_positions"
            if reason:
                req.pending = 0
                self._finish(req, reason)
                done.append(req)
        return done

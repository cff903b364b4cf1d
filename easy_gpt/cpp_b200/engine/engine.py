"""GptEngine: the Python entry point.  Token ids in, token ids out.

It mirrors the reference's ``GptEngine::run`` (src/gpt_engine.cpp:33-43): add the
inputs, run the model until every request has ended, hand back the outputs — but
through the scheduler and the one step function, on the device.
"""
from __future__ import annotations

import tempfile
from pathlib import Path
from typing import List, Optional, Sequence

import time

import torch

from .. import log
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .model import Model
from .scheduler import Request, Scheduler, SchedulerOptions
from .step import StepEntry, StepRunner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def max_new_tokens_from_max_steps(max_steps: int, prompt_len: int) -> int:
    """--max-steps caps prompt + generated tokens; at least one token is generated
    (src/continuous_batch_server.cpp:313)."""
    return max(1, max_steps - prompt_len + 1)


class GptEngine:
    def __init__(self, model_dir, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 cache_tokens: Optional[int] = None, max_active: int = 16, prefill_batch: int = 4,
                 max_batch_tokens: int = 2048, chunk_size: int = 512, max_tokens_per_request: Optional[int] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("GptEngine needs a CUDA device; there is no CPU path")
        torch_dtype = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.model = Model.from_dir(model_dir, device=device, dtype=torch_dtype)
        spec = self.model.spec
        if cache_tokens is None:
            cache_tokens = max_active * min(spec.max_positions, 4096)
        num_pages = -(-cache_tokens // page_size)
        self.runner = StepRunner(self.model, page_size, num_pages, max_slots=max_active,
                                 max_tokens_per_request=max_tokens_per_request or min(spec.max_positions, num_pages * page_size))
        self.scheduler = Scheduler(self.runner.cache, SchedulerOptions(
            max_batch_tokens=max_batch_tokens, chunk_size=chunk_size, max_active=max_active, prefill_batch=prefill_batch,
            eos_token_id=spec.eos_token_id, max_positions=spec.max_positions))
        self.sampler = Sampler(self.model.device, max_rows=max_active)
        self._inflight = None          # (batch, device tokens, host copy in progress, request id -> row) of the last step
        self._added_at = {}            # request id -> time it was added (for the completion line)
        log.info(f"engine on {self.model.device}: {spec.architecture}, {len(spec.run_order)} layers, {dtype}, pages of {page_size} "
                 f"tokens, {num_pages} pages, up to {max_active} live requests")

    # -- requests -------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    max_new_tokens: Optional[int] = None, max_steps: Optional[int] = None) -> Request:
        params = params or SamplingParams()
        if max_new_tokens is None:
            max_new_tokens = max_new_tokens_from_max_steps(max_steps if max_steps is not None else 100, len(prompt))
        vocab = self.model.spec.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        request = self.scheduler.add(prompt, params, max_new_tokens)
        if log.enabled("info"):
            self._added_at[request.id] = time.perf_counter()
        return request

    def _log_finished(self, finished: List[Request]) -> List[Request]:
        """One line per finished request: tokens and rate (cf. src/continuous_batch_server.cpp:249-256)."""
        for r in finished:
            t0 = self._added_at.pop(r.id, None)
            if t0 is not None and log.enabled("info"):
                seconds = max(time.perf_counter() - t0, 1e-9)
                log.info(f"request {r.id} finished ({r.finish_reason}): {len(r.prompt)} prompt tokens, {len(r.output)} new tokens "
                         f"in {1e3 * seconds:.1f} ms ({len(r.output) / seconds:.1f} tok/s), {r.preemptions} preemptions")
        return finished

    def step(self) -> List[Request]:
        with log.nvtx_range("engine.step"):
            return self._log_finished(self._step())

    def _step(self) -> List[Request]:
        """One scheduler round and one model step.  Returns the requests that finished.

        Decode steps are pipelined: a step is put on the device before the previous step's sampled
        tokens have been read by the host — the device feeds them to itself — and the previous
        tokens are read while the new step runs.  So the host's work hides behind the device's, and
        a request that turns out to have ended (EOS) has one token computed in vain, which is dropped.
        Whenever the next batch needs token ids on the host (a prompt portion of a recomputed
        request, a batch the captured path does not take) the tokens in flight are read first."""
        batch = self.scheduler.schedule()
        finished: List[Request] = []
        if not batch:
            return self._resolve_inflight()
        on_device = [s for s in batch if s.pending]                  # entries whose token is still on the device
        graph = None
        if on_device:
            # the device can feed itself only if every entry is a decode of a token of the step in flight
            all_decode = len(on_device) == len(batch) and all(s.count == 1 and s.samples for s in batch)
            graph, handles = self.runner.decode_graph_for([s.request.id for s in batch]) \
                if (all_decode and self.runner.use_graphs) else (None, None)
            if graph is None:
                # the general path needs every token id on the host: read what is in flight, drop what has ended
                finished += self._resolve_inflight()
                for s in batch:
                    s.pending = 0            # read by now: the token is in the request's output
                kept = [s for s in batch if s.request.state == "running"]
                if len(kept) != len(batch):
                    batch = kept
                    if not batch:
                        return finished
                on_device = []
        if log.enabled("debug"):
            log.debug(f"step {self.scheduler.stats.steps}: " + ", ".join(
                f"{s.request.id}[{s.start}:{s.start + s.count}]" + ("*" if s.samples else "") for s in batch))
        if on_device:
            logits = self._launch_on_device_tokens(batch, graph, handles)
        else:
            entries = [StepEntry(s.request.id, s.request.token_slice(s.start, s.count),
                                 [s.count - 1] if s.samples else []) for s in batch]
            logits = self.runner.run(entries, check=False, commit=False)
        self.scheduler.launched(batch)
        sampling = [s for s in batch if s.samples]
        previous = self._inflight
        self._inflight = None
        if sampling and log.enabled("trace"):
            # the five best tokens of every sampled row (cf. src/models/gpt_model.cpp:76-110); costs a synchronisation
            top = torch.topk(logits[:len(sampling)] if logits.shape[0] >= len(sampling) else logits, 5, dim=-1)
            for s, ids, vals in zip(sampling, top.indices.tolist(), top.values.tolist()):
                log.trace(f"request {s.request.id} top-5: " + ", ".join(f"{i}:{v:.3f}" for i, v in zip(ids, vals)))
        if sampling:
            dev = self.sampler.sample(logits, [s.request.params for s in sampling], [s.request.id for s in sampling],
                                      [len(s.request.output) + s.pending for s in sampling])
            self._inflight = (batch, dev, self.sampler.to_host_async(dev), {s.request.id: i for i, s in enumerate(sampling)})
        if previous is not None:
            finished += self._resolve(previous)
        return finished

    def _launch_on_device_tokens(self, batch, graph, handles):
        """A decode step whose input tokens are the previous step's samples, still on the device."""
        _, prev_dev, _, prev_rows = self._inflight
        rows = [prev_rows[s.request.id] for s in batch]
        for s in batch:
            self.runner.cache.reserve(s.request.id, 1)
        if rows == list(range(len(rows))) and len(rows) == prev_dev.numel():
            tokens = prev_dev
        else:
            index = torch.tensor(rows, dtype=torch.int64).pin_memory().to(self.model.device, non_blocking=True)
            tokens = prev_dev.index_select(0, index)
        graph.set_tokens_from_device(tokens)
        logits = graph.replay([s.request.id for s in batch], None, tokens_on_device=True, handles=handles)
        self.runner.graph_replays += 1
        self.runner.last_graph = graph
        return logits[:len(batch)]

    def _resolve(self, inflight) -> List[Request]:
        batch, _, pending_copy, _ = inflight
        return self.scheduler.resolve(batch, pending_copy())

    def sync(self) -> List[Request]:
        """Reads the tokens of the step in flight, if any; returns the requests that finished with them."""
        return self._resolve_inflight()

    def _resolve_inflight(self) -> List[Request]:
        if self._inflight is None:
            return []
        inflight, self._inflight = self._inflight, None
        return self._resolve(inflight)

    def run_to_completion(self) -> None:
        while self.scheduler.has_work():
            before = self.scheduler.stats.steps
            done = self.step()
            if self.scheduler.stats.steps == before and not done and self._inflight is None and self.scheduler.has_work():
                raise RuntimeError("the scheduler made no progress although requests are waiting")
        self._log_finished(self._resolve_inflight())
        self.runner.check_status()

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: Optional[int] = None,
                 max_steps: Optional[int] = None, temperature: float = 0.8, top_p: float = 0.95, top_k: int = 20,
                 seed: int = 42, greedy: bool = False) -> List[List[int]]:
        """Generates for every prompt (lists of token ids) and returns the new tokens of each."""
        params = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, seed=seed, greedy=greedy)
        requests = [self.add_request(p, params, max_new_tokens, max_steps) for p in prompts]
        self.run_to_completion()
        errors = [(r.id, r.error) for r in requests if r.error]
        outputs = [list(r.output) for r in requests]
        for r in requests:
            self.scheduler.forget(r)         # their records are not needed any more: the engine may live long
        if errors:
            raise RuntimeError(f"request {errors[0][0]}: {errors[0][1]}")
        return outputs


def engine_with_random_weights(config: dict, seed: int, folder=None, store_dtype="bfloat16", **engine_options) -> GptEngine:
    """Writes a model folder with random weights for ``config`` and opens an engine on it."""
    from ..weights.random_init import write_random_model

    folder = Path(folder or tempfile.mkdtemp(prefix="easy_gpt_random_"))
    write_random_model(folder, config, seed, store_dtype=store_dtype)
    return GptEngine(folder, **engine_options)

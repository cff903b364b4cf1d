"""A model put together from a :class:`ModelSpec`: parts built by kind from the
registries, weights loaded by name, and a forward over one step's batch that
follows the spec's run order.  (The reference's counterpart is
``GptModel::forward_logits``, src/models/gpt_model.cpp:310-333.)
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import torch

from .. import architectures, parts  # noqa: F401  (registers what the framework ships)
from ..cache.manager import CacheManager
from ..config.spec import LayerSpec, ModelSpec
from .. import kernels
from ..parts.base import FollowingNorm, PendingNorm, StepContext
from ..registry import model_spec_from_config, part_class
from ..weights.loader import load_checked


class Block:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)) with the additions folded
    into the next norm (src/models/block.cpp:23-29)."""

    def __init__(self, spec: LayerSpec):
        position = None
        if spec.position is not None:
            position = part_class("position", spec.position.kind)(spec.position.params, spec.position.prefix)
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm.params, spec.mixer_norm.prefix)
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer.params, spec.mixer.prefix, position)
        self.ff_norm = part_class("norm", spec.feed_forward_norm.kind)(spec.feed_forward_norm.params,
                                                                      spec.feed_forward_norm.prefix)
        self.feed_forward = part_class("feed_forward", spec.feed_forward.kind)(spec.feed_forward.params,
                                                                               spec.feed_forward.prefix)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    @staticmethod
    def _offer(part, norm, pending, ctx, fused_rows):
        """The add and norm after ``part`` as an offer to it, where the part fuses such things, the norm is a plain
        RMSNorm and the step is small enough for the decode kernels."""
        if (part.fuses_following_norm and norm is not None and norm.rms_parameters() is not None
                and ctx.dtype == torch.bfloat16 and 0 < ctx.num_tokens <= fused_rows):
            return dict(follow=FollowingNorm(norm, pending))
        return {}

    def forward(self, residual, spare, delta, ctx: StepContext, cache, work, next_norm=None):
        """Returns (residual, spare, delta): the buffer that now holds the residual
        stream, the other one, and the feed-forward's output still to be added (or the
        PreNormed it left for ``next_norm``, the norm that runs after this block)."""
        fused_rows = kernels.fused_norm_max_tokens(residual.shape[1])
        pending = PendingNorm(self.mixer_norm, residual, delta, spare, work, max_fused_rows=fused_rows)
        delta = self.mixer.forward(pending if self.mixer.accepts_pending_norm else pending.materialize(), ctx, cache,
                                   **self._offer(self.mixer, self.ff_norm, pending, ctx, fused_rows))
        assert pending.consumed, "a mixer that accepts a pending norm must use it"
        residual, spare = pending.residual_after, pending.spare_after
        pending = PendingNorm(self.ff_norm, residual, delta, spare, work, max_fused_rows=fused_rows)
        delta = self.feed_forward.forward(pending if self.feed_forward.accepts_pending_norm else pending.materialize(), ctx,
                                          **self._offer(self.feed_forward, next_norm, pending, ctx, fused_rows))
        assert pending.consumed, "a feed-forward that accepts a pending norm must use it"
        return pending.residual_after, pending.spare_after, delta


class Model:
    def __init__(self, spec: ModelSpec, device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        self.embedding = part_class("head", spec.embedding.kind)(spec.embedding.params, spec.embedding.prefix)
        self.blocks: List[Block] = [Block(l) for l in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm.prefix)
        self.lm_head = part_class("head", spec.lm_head.kind)(spec.lm_head.params, spec.lm_head.prefix)

    # -- weights ---------------------------------------------------------------
    def all_parts(self):
        out = [self.embedding]
        for b in self.blocks:
            out += b.parts()
        return out + [self.final_norm, self.lm_head]

    @property
    def capturable(self) -> bool:
        """Whether decode steps of this model may be captured in a CUDA graph: every part says so."""
        parts = self.all_parts() + [b.mixer.position for b in self.blocks if b.mixer.position is not None]
        return all(p.capturable for p in parts)

    def tensor_requests(self):
        reqs = []
        for p in self.all_parts():
            reqs += p.tensor_requests()
        return reqs

    def load_weights(self, model_file) -> None:
        tensors = load_checked(model_file, self.tensor_requests())
        self.embedding.load(tensors, self.device, self.dtype)
        for b in self.blocks:
            for p in b.parts():
                p.load(tensors, self.device, self.dtype)
        self.final_norm.load(tensors, self.device, self.dtype)
        self.lm_head.load(tensors, self.device, self.dtype, tied_table=self.embedding.table)
        self._wire_prefetch_hints()

    def _wire_prefetch_hints(self) -> None:
        """Tells every part which weights are streamed right after it (by the run order)."""
        order = []
        for e in self.spec.run_order:
            b = self.blocks[e.layer]
            order += [b.mixer, b.feed_forward]
        order.append(self.lm_head)
        for part, nxt in zip(order, order[1:]):
            if not part.prefetch_hints:
                part.prefetch_hints = tuple(nxt.streamed_weights())

    @staticmethod
    def from_dir(model_dir, device="cuda:0", dtype=torch.bfloat16) -> "Model":
        model_dir = Path(model_dir)
        cfg_path = model_dir / "config.json"
        if not cfg_path.is_file():
            raise FileNotFoundError(f"no config.json in {model_dir}")
        spec = model_spec_from_config(json.loads(cfg_path.read_text()))
        model = Model(spec, device, dtype)
        model.load_weights(model_dir / "model.safetensors")
        return model

    # -- caches -------------------------------------------------------------------
    def cache_needs(self) -> Dict[int, object]:
        """cache id -> what the entry that writes it needs."""
        needs = {}
        for e in self.spec.run_order:
            if e.writes_cache:
                needs[e.cache] = self.blocks[e.layer].mixer.cache_need()
        for e in self.spec.run_order:
            if not e.writes_cache and self.blocks[e.layer].mixer.cache_need() != needs[e.cache]:
                raise ValueError(f"a run entry of layer {e.layer} reads cache {e.cache}, whose shape differs from its own")
        return needs

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a step reads once each (embedding rows not counted)."""
        total = 0
        for e in self.spec.run_order:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts())
        return total + self.final_norm.weight_bytes() + self.lm_head.weight_bytes()

    # -- forward ------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: CacheManager, logit_rows: Optional[torch.Tensor],
                all_rows: bool = False) -> Optional[torch.Tensor]:
        """Runs the batch through every run entry; returns float32 logits at
        ``logit_rows`` (token indices into the batch), or None when none is wanted.
        ``all_rows``: logit_rows is 0..T-1 in order (a decode step), no gather needed."""
        T, H = ctx.num_tokens, self.spec.hidden_size
        ctx.scratch.clear()
        residual = torch.empty((T, H), device=self.device, dtype=torch.float32)
        spare = torch.empty((T, H), device=self.device, dtype=torch.float32)
        work = torch.empty((T, H), device=self.device, dtype=self.dtype)
        self.embedding.forward(ctx.token_ids, residual, ctx.status)
        delta = None
        order = self.spec.run_order
        for i, e in enumerate(order):
            next_norm = self.blocks[order[i + 1].layer].mixer_norm if i + 1 < len(order) else self.final_norm
            residual, spare, delta = self.blocks[e.layer].forward(residual, spare, delta, ctx,
                                                                  cache.view(e.cache, e.writes_cache), work, next_norm)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        pending = PendingNorm(self.final_norm, residual, delta, spare, work, rows=None if all_rows else logit_rows,
                              max_fused_rows=kernels.fused_norm_max_tokens(H))
        return self.lm_head.forward(pending if self.lm_head.accepts_pending_norm else pending.materialize(), status=ctx.status)

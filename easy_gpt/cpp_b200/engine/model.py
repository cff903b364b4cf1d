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
from .. import kernels, log
from ..parts.base import FollowingNorm, PendingNorm, StepContext
from ..registry import model_spec_from_config, part_class
from ..weights.loader import load_checked


class SubLayer:
    """One built sub-layer of a block: the part, the norm in front of it or behind it, and an optional
    norm on its output (see ``SubLayerSpec``)."""

    def __init__(self, spec, position):
        build = lambda role, ps: part_class(role, ps.kind)(ps.params, ps.prefix)
        self.role = spec.role
        self.placement = spec.norm_placement
        self.norm = build("norm", spec.norm) if spec.norm is not None else None
        self.output_norm = build("norm", spec.output_norm) if spec.output_norm is not None else None
        cls = part_class(spec.role, spec.part.kind)
        self.part = cls(spec.part.params, spec.part.prefix, position) if spec.role == "mixer" else cls(spec.part.params, spec.part.prefix)
        # x = x + part(norm(x)) with nothing behind the part: the shape whose add and norm the parts may fuse
        self.plain_pre_norm = self.norm is not None and self.placement == "pre" and self.output_norm is None

    def parts(self):
        return [p for p in (self.norm, self.part, self.output_norm) if p is not None]


class Block:
    """A layer: its residual sub-layers in order.  For the pre-norm shape x += mixer(norm1(x));
    x += feed_forward(norm2(x)) (src/models/block.cpp:23-29) every addition is folded into the norm
    that follows it, or into the kernels around it where the parts offer that.  Other shapes (a norm
    behind the part, a norm on the part's output, no norm, no feed-forward) run the same parts with
    the additions and norms as kernels of their own."""

    def __init__(self, spec: LayerSpec):
        position = None
        if spec.position is not None:
            position = part_class("position", spec.position.kind)(spec.position.params, spec.position.prefix)
        self.sublayers = [SubLayer(s, position) for s in spec.sublayers]
        mixers = [s.part for s in self.sublayers if s.role == "mixer"]
        self.mixer = mixers[0] if mixers else None
        self.position = position

    def parts(self):
        return [p for s in self.sublayers for p in s.parts()]

    @property
    def first_norm(self):
        """The norm that a fused add + norm in front of this layer would have to be: the first sub-layer's,
        if that is a plain pre-norm one; else None (nothing in front may prepare it)."""
        first = self.sublayers[0]
        return first.norm if first.plain_pre_norm else None

    @staticmethod
    def _offer(part, norm, pending, ctx, fused_rows):
        """The add and norm after ``part`` as an offer to it, where the part fuses such things, the norm is a plain
        RMSNorm and the step is small enough for the decode kernels."""
        if (part.fuses_following_norm and norm is not None and norm.rms_parameters() is not None
                and ctx.dtype == torch.bfloat16 and 0 < ctx.num_tokens <= fused_rows):
            return dict(follow=FollowingNorm(norm, pending))
        return {}

    @staticmethod
    def _settle(residual, delta):
        """The residual stream with a delta that was still to be added (float32, in place)."""
        if delta is not None:
            residual.add_(delta)
        return residual

    def forward(self, residual, spare, delta, ctx: StepContext, cache, work, next_norm=None):
        """Returns (residual, spare, delta): the buffer that now holds the residual stream, the other
        one, and what the last sub-layer left still to be added (its output, or the PreNormed it
        prepared for ``next_norm``, the norm that runs after this block; None: nothing is pending)."""
        fused_rows = kernels.fused_norm_max_tokens(residual.shape[1])
        subs = self.sublayers
        for i, sub in enumerate(subs):
            following = subs[i + 1].norm if i + 1 < len(subs) and subs[i + 1].plain_pre_norm else \
                (next_norm if i + 1 == len(subs) else None)
            args = (ctx, cache) if sub.role == "mixer" else (ctx,)
            if log.NVTX:
                torch.cuda.nvtx.range_push(f"{sub.role}:{type(sub.part).__name__}")
            try:
                residual, spare, delta = self._run_sublayer(sub, following, args, residual, spare, delta, ctx, work, fused_rows)
            finally:
                if log.NVTX:
                    torch.cuda.nvtx.range_pop()
        return residual, spare, delta

    def _run_sublayer(self, sub, following, args, residual, spare, delta, ctx, work, fused_rows):
        if sub.plain_pre_norm:
            pending = PendingNorm(sub.norm, residual, delta, spare, work, max_fused_rows=fused_rows)
            delta = sub.part.forward(pending if sub.part.accepts_pending_norm else pending.materialize(), *args,
                                     **self._offer(sub.part, following, pending, ctx, fused_rows))
            assert pending.consumed, "a part that accepts a pending norm must use it"
            return pending.residual_after, pending.spare_after, delta
        # the general shapes: the stream is settled first, every norm is a kernel of its own
        residual = self._settle(residual, delta)
        if sub.norm is not None and sub.placement == "pre":
            x = sub.norm.forward(residual, None, work)
        else:
            x = work.copy_(residual)
        delta = sub.part.forward(x, *args)
        if sub.output_norm is not None:
            delta = self._normalised(sub.output_norm, delta, spare, like=work)
        if sub.norm is not None and sub.placement == "post":
            # x = norm(x + part(x)): the normalised sum is the new residual stream
            sub.norm.forward(residual, delta, spare)
            residual, spare = spare, residual
            delta = None
        return residual, spare, delta

    @staticmethod
    def _normalised(norm, delta, scratch_f32, like):
        """norm(delta) in the compute dtype (a norm on a part's output)."""
        scratch_f32.copy_(delta)
        out = torch.empty_like(like)
        return norm.forward(scratch_f32, None, out)


class Model:
    def __init__(self, spec: ModelSpec, device, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        self.embedding = part_class("head", spec.embedding.kind)(spec.embedding.params, spec.embedding.prefix)
        self.embedding_position = None
        if spec.embedding_position is not None:
            ep = spec.embedding_position
            self.embedding_position = part_class("position", ep.kind)(ep.params, ep.prefix)
        self.blocks: List[Block] = [Block(l) for l in spec.layers]
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm.prefix)
        self.lm_head = part_class("head", spec.lm_head.kind)(spec.lm_head.params, spec.lm_head.prefix)

    # -- weights ---------------------------------------------------------------
    def all_parts(self):
        out = [self.embedding] + ([self.embedding_position] if self.embedding_position is not None else [])
        for b in self.blocks:
            out += b.parts()
        return out + [self.final_norm, self.lm_head]

    @property
    def capturable(self) -> bool:
        """Whether decode steps of this model may be captured in a CUDA graph: every part says so."""
        parts = self.all_parts() + [b.position for b in self.blocks if b.position is not None]
        return all(p.capturable for p in parts)

    def tensor_requests(self):
        reqs = []
        for p in self.all_parts():
            reqs += p.tensor_requests()
        return reqs

    def load_weights(self, model_file) -> None:
        tensors = load_checked(model_file, self.tensor_requests())
        self.embedding.load(tensors, self.device, self.dtype)
        if self.embedding_position is not None:
            self.embedding_position.load(tensors, self.device, self.dtype)
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
            order += [s.part for s in self.blocks[e.layer].sublayers]
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
        need_of = lambda layer: self.blocks[layer].mixer.cache_need() if self.blocks[layer].mixer is not None else None
        for e in self.spec.run_order:
            if e.writes_cache:
                needs[e.cache] = need_of(e.layer)
        for e in self.spec.run_order:
            if not e.writes_cache and need_of(e.layer) != needs[e.cache]:
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
        self.embedding.forward(ctx, residual)
        if self.embedding_position is not None:
            self.embedding_position.add_to_embedding(residual, ctx)
        delta = None
        order = self.spec.run_order
        for i, e in enumerate(order):
            next_norm = self.blocks[order[i + 1].layer].first_norm if i + 1 < len(order) else self.final_norm
            residual, spare, delta = self.blocks[e.layer].forward(residual, spare, delta, ctx,
                                                                  cache.view(e.cache, e.writes_cache), work, next_norm)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        pending = PendingNorm(self.final_norm, residual, delta, spare, work, rows=None if all_rows else logit_rows,
                              max_fused_rows=kernels.fused_norm_max_tokens(H))
        return self.lm_head.forward(pending if self.lm_head.accepts_pending_norm else pending.materialize(), status=ctx.status)

"""Grouped-query attention over the paged cache.

Per token: q, k, v = x Wq^T + bq, ... (src/models/self_attn.cpp:225-227) as ONE
product with the three weights stacked; q and k are changed by the layer's position
encoding (a half rotation is applied by the kernel that also stores k, v in the
cache; another encoding changes q and k itself; none is fine too); every query head h attends the keys of KV head
h / (NH/NKV) of its own request up to its own position (optionally only the last
``window`` of them); the heads are concatenated head-major and projected by Wo
(src/models/self_attn.cpp:255-258).  Scale 1/sqrt(head_dim) (:253).

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, out_bias,
window (None = all keys).
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import CacheView, Mixer, PagedKVNeed, PendingNorm, StepContext
from .linear import Linear


class Attention(Mixer):
    capturable = True

    def __init__(self, params, prefix, position=None):
        super().__init__(params, prefix, position)
        p = params
        self.hidden = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.out_bias = bool(p.get("out_bias", False))
        self.window = p.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive")
        if not 0 < self.head_dim <= kernels.MAX_HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} is outside what the attention kernels take (1..{kernels.MAX_HEAD_DIM})")
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.qkv = self.out = None

    # -- weights ----------------------------------------------------------
    def tensor_requests(self):
        q_out, kv_out = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        reqs = [TensorRequest.matrix(f"{self.prefix}.q_proj.weight", q_out, self.hidden),
                TensorRequest.matrix(f"{self.prefix}.k_proj.weight", kv_out, self.hidden),
                TensorRequest.matrix(f"{self.prefix}.v_proj.weight", kv_out, self.hidden),
                TensorRequest.matrix(f"{self.prefix}.o_proj.weight", self.hidden, q_out)]
        if self.qkv_bias:
            reqs += [TensorRequest.vector(f"{self.prefix}.q_proj.bias", q_out),
                     TensorRequest.vector(f"{self.prefix}.k_proj.bias", kv_out),
                     TensorRequest.vector(f"{self.prefix}.v_proj.bias", kv_out)]
        if self.out_bias:
            reqs.append(TensorRequest.vector(f"{self.prefix}.o_proj.bias", self.hidden))
        return reqs

    def load(self, tensors, device, dtype):
        names = [f"{self.prefix}.{n}_proj" for n in "qkv"]
        w = torch.cat([tensors[n + ".weight"].float() for n in names], dim=0)
        b = torch.cat([tensors[n + ".bias"].float().reshape(-1) for n in names]) if self.qkv_bias else None
        self.qkv = Linear(w, b, device, dtype)
        self.out = Linear(tensors[f"{self.prefix}.o_proj.weight"],
                          tensors.get(f"{self.prefix}.o_proj.bias") if self.out_bias else None, device, dtype)
        if self.position is not None:
            self.position.load(tensors, device, dtype)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.out.weight_bytes()

    def streamed_weights(self):
        return [self.qkv.weight, self.out.weight]

    # -- cache ------------------------------------------------------------
    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_dim, self.window)

    # -- forward ----------------------------------------------------------
    accepts_pending_norm = True
    fuses_following_norm = True

    @staticmethod
    def _rotation_table(rot, ctx):
        """cos/sin [T, rotary_dim/2, 2] of this step's positions: computed by the first layer that asks and
        shared by every layer whose rotation has the same key."""
        key = ("rotation table",) + tuple(rot.key) if rot.key else ("rotation table", rot.inv_freq.data_ptr())
        if key not in ctx.scratch:
            ctx.scratch[key] = kernels.rope_table(ctx.positions, rot.inv_freq)
        return ctx.scratch[key]

    def forward(self, x, ctx: StepContext, cache: CacheView, follow=None):
        """x: the normalised input [T, hidden], or a PendingNorm that stands for it.  ``follow``: the add
        and norm that come next; the output product of a decode step takes them over."""
        T = ctx.num_tokens
        tables = ctx.groups[cache.group]
        pending = x if isinstance(x, PendingNorm) else None
        dtype, device = ctx.dtype, ctx.device
        # what the layer's position encoding offers: a half rotation that the kernels apply themselves,
        # or a change of q and k of its own making, or nothing at all (no position encoding)
        rot = self.position.half_rotation() if self.position is not None else None
        if (pending is not None and pending.fusable and cache.writes and rot is not None
                and rot.rotary_dim == self.head_dim and self.head_dim in (16, 32, 64, 128)):
            # decode: add + norm + QKV product + bias + rotation + cache write in one kernel
            q = torch.empty((T, self.num_heads * self.head_dim), device=device, dtype=dtype)
            kernels.gemm_skinny(self.qkv.weight, self.qkv.bias_f32, q, kernels.EPI_QKV_ROPE, tokens=T, norm=pending.fused(),
                                rope=dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                                          positions=ctx.positions, slot_map=tables.slot_map, k_cache=cache.k,
                                          v_cache=cache.v, inv_freq=rot.inv_freq, status=ctx.status))
            qkv = q
        else:
            if pending is not None:
                x = pending.materialize()
            qkv = self.qkv(x, status=ctx.status)
            store = (tables.slot_map, cache.k, cache.v) if cache.writes else (None, None, None)
            if rot is not None and rot.rotary_dim == self.head_dim and self.head_dim % (16 if qkv.dtype == torch.bfloat16 else 8) == 0:
                kernels.rope_cache_table(qkv, self._rotation_table(rot, ctx), *store, self.num_heads, self.num_kv_heads,
                                         self.head_dim, tables.page_size, ctx.status)
            elif rot is not None:
                kernels.rope_cache(qkv, None, ctx.positions, *store, rot.inv_freq, self.num_heads, self.num_kv_heads,
                                   self.head_dim, rot.rotary_dim, tables.page_size, ctx.status)
            else:
                if self.position is not None:
                    q_width, k_width = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
                    self.position.apply_to_query_key(qkv[:, :q_width].view(T, self.num_heads, self.head_dim),
                                                     qkv[:, q_width:q_width + k_width].view(T, self.num_kv_heads, self.head_dim), ctx)
                kernels.rope_cache(qkv, None, ctx.positions, *store, None, self.num_heads, self.num_kv_heads,
                                   self.head_dim, 0, tables.page_size, ctx.status)
        attn = torch.empty((T, self.num_heads * self.head_dim), device=device, dtype=dtype)
        longest = ctx.max_context_len if self.window is None else min(ctx.max_context_len, self.window + 255)
        if ctx.query_tiles is not None and kernels.attention_prefill_takes(dtype, self.head_dim, tables.page_size):
            # prompt portions: tiles of query tokens against the cache, on the tcgen05 tensor cores when
            # the portions are long enough to fill their 128-row tiles
            tensor_core = (kernels.TCGEN05_ATTENTION and ctx.max_query_len >= kernels.TCGEN05_ATTENTION_MIN_QUERY
                           and kernels.attention_prefill_tcgen05_takes(dtype, self.head_dim, tables.page_size))
            if tensor_core:
                parts, part_tiles = kernels.attention_prefill_parts(ctx.query_tiles.shape[0], self.num_heads, self.head_dim)
                kernels.attention_prefill_tcgen05(
                    qkv, cache.k, cache.v, tables.block_table, ctx.positions, ctx.query_tiles, attn, self.num_heads,
                    self.num_kv_heads, self.head_dim, self.window, self.scale, ctx.status, parts=parts, part_tiles=part_tiles)
            else:
                kernels.attention_prefill(qkv, cache.k, cache.v, tables.block_table, ctx.positions, ctx.query_tiles, attn,
                                          self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale,
                                          ctx.status)
            if ctx.small_tokens is not None:
                # the decoded tokens beside them: token by token, split over their keys
                count = ctx.small_tokens.numel()
                kernels.attention_paged(qkv, cache.k, cache.v, tables.block_table, ctx.token_seq, ctx.positions, attn,
                                        self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale,
                                        kernels.attention_paged_splits(count, self.num_heads, self.num_kv_heads, longest, self.head_dim),
                                        ctx.status, token_list=ctx.small_tokens)
        elif kernels.attention_paged_takes(dtype, self.head_dim, tables.page_size):
            splits = kernels.attention_paged_splits(T, self.num_heads, self.num_kv_heads, longest, self.head_dim)
            kernels.attention_paged(qkv, cache.k, cache.v, tables.block_table, ctx.token_seq, ctx.positions, attn,
                                    self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale, splits,
                                    ctx.status, prefetch=self._hint(0) if T <= kernels.SKINNY_MAX_TOKENS else None,
                                    seq_context=ctx.seq_context)
        else:
            kernels.attention_generic(qkv, cache.k, cache.v, tables.block_table, ctx.token_seq, ctx.positions, attn,
                                      self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale,
                                      ctx.status)
        if follow is not None and self.out.takes_following_norm(attn):
            return self.out.with_following_norm(attn, follow, prefetch=self._hint(1), status=ctx.status)
        return self.out(attn, prefetch=self._hint(1), status=ctx.status)


register_part("mixer", "attention", Attention)

"""SwiGLU feed-forward: down( up(x) * silu(gate(x)) ) (src/models/mlp.cpp:41-49).
gate and up become one product whose weight rows are interleaved (gate_0, up_0,
gate_1, up_1, ...), so that every tile of the product holds both halves of the
outputs it covers and the activation can run in the product's epilogue.
Parameters: hidden_size, intermediate_size, bias."""
from __future__ import annotations

import torch

from .. import kernels
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import FeedForward, PendingNorm
from .linear import Linear


class SwiGLU(FeedForward):
    capturable = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", False))
        self.gate_up = self.down = None

    def tensor_requests(self):
        reqs = [TensorRequest.matrix(f"{self.prefix}.gate_proj.weight", self.inter, self.hidden),
                TensorRequest.matrix(f"{self.prefix}.up_proj.weight", self.inter, self.hidden),
                TensorRequest.matrix(f"{self.prefix}.down_proj.weight", self.hidden, self.inter)]
        if self.bias:
            reqs += [TensorRequest.vector(f"{self.prefix}.gate_proj.bias", self.inter),
                     TensorRequest.vector(f"{self.prefix}.up_proj.bias", self.inter),
                     TensorRequest.vector(f"{self.prefix}.down_proj.bias", self.hidden)]
        return reqs

    def load(self, tensors, device, dtype):
        p = self.prefix
        w = torch.stack([tensors[f"{p}.gate_proj.weight"].float(), tensors[f"{p}.up_proj.weight"].float()], dim=1)
        w = w.reshape(2 * self.inter, self.hidden)
        b = torch.stack([tensors[f"{p}.gate_proj.bias"].float().reshape(-1),
                         tensors[f"{p}.up_proj.bias"].float().reshape(-1)], dim=1).reshape(-1) if self.bias else None
        self.gate_up = Linear(w, b, device, dtype)
        self.down = Linear(tensors[f"{p}.down_proj.weight"], tensors.get(f"{p}.down_proj.bias") if self.bias else None,
                           device, dtype)

    def weight_bytes(self):
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def streamed_weights(self):
        return [self.gate_up.weight, self.down.weight]

    accepts_pending_norm = True
    fuses_following_norm = True

    def forward(self, x, ctx, follow=None):
        """x: the normalised input [T, hidden], or a PendingNorm that stands for it.  ``follow``: the add
        and norm that come next; the down product of a decode step takes them over."""
        T = ctx.num_tokens
        act = torch.empty((T, self.inter), device=ctx.device, dtype=ctx.dtype)
        if isinstance(x, PendingNorm) and x.fusable:
            # decode: add + norm + gate/up product + SwiGLU in one kernel
            kernels.gemm_skinny(self.gate_up.weight, self.gate_up.bias_f32, act, kernels.EPI_SWIGLU, tokens=T,
                                prefetch=self._hint(0), status=ctx.status, norm=x.fused())
        else:
            if isinstance(x, PendingNorm):
                x = x.materialize()
            if kernels.gemm_skinny_takes(ctx.dtype, T, self.hidden):
                kernels.gemm_skinny(self.gate_up.weight, self.gate_up.bias_f32, act, kernels.EPI_SWIGLU, x=x,
                                    prefetch=self._hint(0))
            elif kernels.gemm_tcgen05_few_takes(ctx.dtype, T, 2 * self.inter, self.hidden) and x.stride(0) % 8 == 0:
                # the larger decode batches and short portions: tcgen05 product over narrow column tiles, SwiGLU in its epilogue
                kernels.gemm_tcgen05_few(x, self.gate_up.weight, self.gate_up.bias_f32, act, ctx.status, epilogue=kernels.EPI_SWIGLU)
            elif kernels.gemm_tcgen05_wide_takes(ctx.dtype, T, 2 * self.inter, self.hidden):
                # prompts: the product on the tcgen05 tensor cores (persistent 128 x 256 tiles) with SwiGLU in its epilogue
                kernels.gemm_tcgen05(x, self.gate_up.weight, self.gate_up.bias_f32, act, ctx.status, swiglu_epilogue=True,
                                     pair=kernels.USE_TCGEN05_PAIR)
            else:
                kernels.swiglu(self.gate_up(x), act)
        if follow is not None and self.down.takes_following_norm(act):
            return self.down.with_following_norm(act, follow, prefetch=self._hint(1), status=ctx.status)
        return self.down(act, prefetch=self._hint(1), status=ctx.status)


register_part("feed_forward", "swiglu", SwiGLU)

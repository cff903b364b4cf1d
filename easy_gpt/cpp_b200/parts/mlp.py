"""SwiGLU feed-forward: down( up(x) * silu(gate(x)) ) (src/models/mlp.cpp:41-49).
gate and up are stacked into one product; parameters: hidden_size,
intermediate_size, bias."""
from __future__ import annotations

import torch

from .. import kernels
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
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
        w = torch.cat([tensors[f"{p}.gate_proj.weight"].float(), tensors[f"{p}.up_proj.weight"].float()], dim=0)
        b = torch.cat([tensors[f"{p}.gate_proj.bias"].float().reshape(-1),
                       tensors[f"{p}.up_proj.bias"].float().reshape(-1)]) if self.bias else None
        self.gate_up = Linear(w, b, device, dtype)
        self.down = Linear(tensors[f"{p}.down_proj.weight"], tensors.get(f"{p}.down_proj.bias") if self.bias else None,
                           device, dtype)

    def weight_bytes(self):
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def forward(self, x, ctx):
        gu = self.gate_up(x)
        act = torch.empty((x.shape[0], self.inter), device=x.device, dtype=x.dtype)
        kernels.swiglu(gu, act)
        return self.down(act)


register_part("feed_forward", "swiglu", SwiGLU)

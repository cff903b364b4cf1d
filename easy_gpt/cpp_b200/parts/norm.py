"""RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)) (src/models/norm.cpp:46-60), eps
a parameter (the reference fixes 1e-6, src/models/norm.cpp:41), fused with the
float32 residual add."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..registry import register_part
from ..weights.loader import TensorRequest
from .base import Norm


class RMSNorm(Norm):
    capturable = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.gain = None

    def tensor_requests(self):
        return [TensorRequest.vector(self.prefix + ".weight", self.size)]

    def load(self, tensors, device, dtype):
        # gains are used in float32 whatever precision they were stored in
        self.gain = tensors[self.prefix + ".weight"].to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    def weight_bytes(self):
        return self.gain.numel() * 4

    def rms_parameters(self):
        return self.gain, self.eps

    def forward(self, residual, delta, out, rows: Optional[torch.Tensor] = None):
        kernels.add_rmsnorm(residual, delta, self.gain, out, self.eps, rows)
        n = rows.numel() if rows is not None else residual.shape[0]
        return out[:n]


register_part("norm", "rmsnorm", RMSNorm)

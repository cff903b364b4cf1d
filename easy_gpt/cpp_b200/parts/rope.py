"""Rotary position encoding, half rotation over ``rotary_dim`` dimensions of each
head (src/ops.cpp:404-421).  The table inv_freq[k] = theta^(-2k/rotary_dim)
(src/ops.cpp:172-177) is built once on the host, in double, rounded to float32;
the kernels multiply it by the float32 position and take the accurate cosf/sinf.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import kernels
from ..registry import register_part
from .base import HalfRotation, PositionEncoding


class RotaryEncoding(PositionEncoding):
    capturable = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        if self.theta <= 0:
            raise ValueError("rope theta must be > 0")
        self.inv_freq = None

    @staticmethod
    def inverse_frequencies(rotary_dim: int, theta: float) -> torch.Tensor:
        k = np.arange(rotary_dim // 2, dtype=np.float64)
        return torch.from_numpy((1.0 / np.power(np.float64(theta), 2.0 * k / rotary_dim)).astype(np.float32))

    def load(self, tensors, device, dtype):
        self.inv_freq = self.inverse_frequencies(self.rotary_dim, self.theta).to(device)

    def half_rotation(self) -> HalfRotation:
        return HalfRotation(self.inv_freq, self.rotary_dim, key=("rope", self.theta, self.rotary_dim))


register_part("position", "rope", RotaryEncoding)

"""Weights by tensor name, checked against what the model's parts declare.

Every part lists the tensors it needs (:class:`TensorRequest`).  The loader
compares that manifest with the file and raises ONE :class:`WeightError` that
lists every missing tensor, every unexpected tensor and every wrong shape.
(The reference collects missing keys the same way,
src/models/model_param_validation.cpp:152-154, checks shapes one by one,
:156-195, and only warns about leftovers, :198-218.)
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = []
        if self.missing:
            lines.append("Missing required model weights: " + ", ".join(self.missing))
        if self.unexpected:
            lines.append("Unexpected tensors in the file: " + ", ".join(self.unexpected))
        for name, expected, got in self.wrong_shape:
            lines.append(f"Invalid tensor shape for key '{name}': expected {expected}, got {list(got)}")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorRequest:
    name: str
    shapes: Tuple[Tuple[int, ...], ...]      # every accepted shape; the first is the canonical one
    optional: bool = False

    @staticmethod
    def matrix(name, rows, cols, optional=False):
        return TensorRequest(name, ((rows, cols),), optional)

    @staticmethod
    def vector(name, n, optional=False):
        # a [n, 1] vector is accepted like [n] (src/models/model_param_validation.cpp:62-74)
        return TensorRequest(name, ((n,), (n, 1)), optional)

    def describe(self) -> str:
        return " or ".join(str(list(s)) for s in self.shapes)


def check_manifest(requests: Sequence[TensorRequest], available: Dict[str, Tuple[int, ...]]) -> None:
    missing, wrong = [], []
    wanted = set()
    for r in requests:
        wanted.add(r.name)
        if r.name not in available:
            if not r.optional:
                missing.append(r.name)
            continue
        if tuple(available[r.name]) not in r.shapes:
            wrong.append((r.name, r.describe(), available[r.name]))
    unexpected = sorted(n for n in available if n not in wanted)
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def load_checked(model_file, requests: Sequence[TensorRequest]) -> Dict[str, torch.Tensor]:
    """Host tensors by name in their stored precision (bfloat16 stays bfloat16,
    a tensor stored in 32 bits stays so, integer tables are int32), vectors
    flattened to one dimension."""
    with SafetensorsFile(Path(model_file)) as f:
        check_manifest(requests, {n: f.shape(n) for n in f.names()})
        out = {}
        for r in requests:
            if r.name in f:
                t = f.tensor(r.name)
                out[r.name] = t.reshape(r.shapes[0]) if tuple(t.shape) != r.shapes[0] else t
        return out

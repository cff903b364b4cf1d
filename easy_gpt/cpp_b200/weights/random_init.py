"""Random-weights mode: writes a model folder (config.json, model.safetensors)
from a configuration and a seed.

Every tensor is drawn from its own generator keyed by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or in which order
they are written.  Matrices and biases are N(0, std) / N(0, bias_std); norm
gains are 1 + N(0, gain_std) (exactly 1 when gain_std is 0).  (The reference has
only unused debug constructors with an unseeded generator, src/utils.cpp:14-15,
src/models/linear.cpp:15-24.)
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Optional

import torch

from ..engine.model import Model
from ..registry import model_spec_from_config
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & ((1 << 63) - 1))
    return g


def random_tensors(config: dict, seed: int, std: float = 0.02, bias_std: Optional[float] = None,
                   gain_std: float = 0.0, store_dtype: str = "bfloat16"):
    """Yields (name, tensor) for every tensor the model of ``config`` asks for."""
    dtype = _STORE[store_dtype]
    bias_std = std if bias_std is None else bias_std
    model = Model(model_spec_from_config(config), "cpu", torch.float32)
    for req in model.tensor_requests():
        shape = req.shapes[0]
        g = _generator(seed, req.name)
        if len(shape) == 1 and req.name.endswith("norm.weight"):
            t = torch.ones(shape)
            if gain_std:
                t = t + torch.randn(shape, generator=g) * gain_std
        elif len(shape) == 1:
            t = torch.randn(shape, generator=g) * bias_std
        else:
            t = torch.randn(shape, generator=g) * std
        yield req.name, t.to(dtype)


def write_random_model(folder, config: dict, seed: int, std: float = 0.02, bias_std: Optional[float] = None,
                       gain_std: float = 0.0, store_dtype: str = "bfloat16") -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    model_spec_from_config(config)                      # refuse a configuration that cannot be run
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(folder / "model.safetensors",
                      random_tensors(config, seed, std, bias_std, gain_std, store_dtype))
    return folder

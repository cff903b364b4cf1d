"""easy_gpt.cpp_b200 — a small, whole, single-GPU inference engine for the Qwen2
dense decoder on B200 (sm_100a): typed configuration, weights by name, layers
put together from parts, a paged cache, one step function, a scheduler,
sampling, and trace replay, on hand-written CUDA kernels."""
from . import architectures, parts  # noqa: F401
from .registry import model_spec_from_config, register_architecture, register_part, resolve_architecture

__all__ = ["model_spec_from_config", "register_architecture", "register_part", "resolve_architecture"]

"""easy_gpt.cpp_b200 — a small, whole, single-GPU inference engine for the Qwen2
dense decoder on B200 (sm_100a): typed configuration, weights by name, layers
put together from parts, a paged cache, one step function, a scheduler,
sampling, and trace replay, on hand-written CUDA kernels.

``native`` is the engine itself (C++, ``csrc/engine``) behind its C interface; ``engine``, ``parts``,
``registry`` and the rest are its PyTorch face, where parts can be written in Python over the same
kernels.  The face is imported on first use, so the native engine runs without PyTorch in the process."""

__all__ = ["model_spec_from_config", "register_architecture", "register_part", "resolve_architecture"]


def __getattr__(name):
    if name in __all__:
        from . import architectures, parts  # noqa: F401  (registers what the framework ships)
        from . import registry

        return getattr(registry, name)
    raise AttributeError(name)

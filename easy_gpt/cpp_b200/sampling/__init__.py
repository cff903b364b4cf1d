"""Sampling: the options of a request, the counter-based uniform numbers, and (for the PyTorch face) the sampler
that launches the kernels.  The sampler is imported on first use, so that the options can be used without PyTorch."""
from .params import GREEDY, SamplingParams
from .rng import uniform

__all__ = ["GREEDY", "Sampler", "SamplingParams", "uniform"]


def __getattr__(name):
    if name == "Sampler":
        from .sampler import Sampler

        return Sampler
    raise AttributeError(name)

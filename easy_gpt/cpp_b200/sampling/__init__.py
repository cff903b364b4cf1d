from .params import GREEDY, SamplingParams
from .rng import uniform

__all__ = ["GREEDY", "SamplingParams", "uniform"]

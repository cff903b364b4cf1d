"""Sampling options of one request.  Names and meanings are the reference's
command line (src/cli_options.cpp:23-47, 105-198): temperature > 0, top_p in
(0, 1], top_k >= 0 (0 disables), seed >= 0, greedy overrides sampling."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 20
    seed: int = 42
    greedy: bool = False

    def __post_init__(self):
        if not self.greedy and not self.temperature > 0.0:
            raise ValueError("Temperature must be greater than 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("Top-p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("Top-k must be >= 0")
        if self.seed < 0:
            raise ValueError("Seed must be >= 0")

    @property
    def is_greedy(self) -> bool:
        # src/sampler.cpp:43-49: greedy when asked for, or when the temperature is not positive
        return self.greedy or self.temperature <= 0.0


GREEDY = SamplingParams(greedy=True)

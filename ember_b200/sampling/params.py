"""Sampling options, with the reference's names, meanings and defaults
(src/backend/backend.hpp:31-37)."""
from __future__ import annotations

from dataclasses import dataclass

GREEDY_THRESHOLD = 1e-5   # temperature <= this means argmax (src/backend/sampling_host.cpp:22)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0    # 0 = greedy
    top_p: float = 1.0
    top_k: int = 0              # 0 = no limit
    min_p: float = 0.0          # drop tokens below min_p * p(best)
    seed: int = 0               # 0 = the engine picks one

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_THRESHOLD

"""Sampling parameters and the per-sequence random keys.

The reference draws with one torch generator shared by everything
(cpmcu/llm.py:55-59, 282-285): ``temperature == 0`` is greedy, otherwise
``multinomial(softmax(logits / temperature))``.  Here a sequence's draw number n uses
the counter-based random value of (seed, sequence key, n), so what a sequence draws
does not depend on which other sequences share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 = greedy (lowest index among equal logits); top_p < 1 keeps the
    smallest set of most likely tokens whose mass reaches top_p."""

    temperature: float = 0.0
    top_p: float = 1.0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0

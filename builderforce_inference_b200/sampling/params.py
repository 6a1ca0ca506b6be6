"""Sampling options, with the reference's names, defaults and meanings
(crates/bfi-runtime/src/sample.rs:10-50; grammar and tool options are out of scope)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SampleParams:
    max_tokens: int = 256          # 0: until the context is full
    temperature: float = 0.0       # <= 0: greedy (lowest index among equal maxima)
    top_k: int = 0                 # 0: off
    top_p: float = 1.0             # 1: off
    min_p: float = 0.0             # 0: off
    repeat_penalty: float = 1.0    # 1: off; applied to every id of prompt + generated, before temperature
    presence_penalty: float = 0.0  # 0: off; subtracted for every seen id, after the repeat penalty
    seed: int = 0

    def validate(self) -> None:
        if self.max_tokens < 0:
            raise ValueError("max_tokens must be >= 0")
        if not self.repeat_penalty > 0.0:
            raise ValueError("repeat_penalty must be > 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_penalties(self) -> bool:
        return abs(self.repeat_penalty - 1.0) > 1.1920929e-07 or self.presence_penalty != 0.0

    @property
    def needs_sort(self) -> bool:
        return (not self.greedy) and (self.top_k > 0 or self.top_p < 1.0)

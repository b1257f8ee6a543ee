"""Sampling options, with the reference's names and defaults (src/types.zig:337-348)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplerParams:
    """temperature <= 0 or greedy means argmax (src/sampler.zig:41).  ``frequency_penalty`` exists in the
    reference's options but its sampler never reads it (src/sampler.zig:55-75); it is kept for the name."""
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    min_p: float = 0.05
    repetition_penalty: float = 1.1
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty_window: int = 64
    seed: int = 42
    greedy: bool = False

    def is_greedy(self) -> bool:
        return self.greedy or self.temperature <= 0.0

    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0

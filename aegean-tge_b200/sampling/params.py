"""Sampling controls with the reference's names, defaults and validation.

``SamplingParams`` mirrors include/tge/models/sampling.hpp:11-27; the checks
are those of ``validate_sampling_params`` (src/models/sampling.cpp:95-127).
The random stream is the reference's xorshift32 (src/models/sampling.cpp:16-28):
seed 0 selects the fixed default 0x9E3779B9, and a draw is ``(state >> 8) / 2**24``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

DEFAULT_SEED = 0x9E3779B9


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # 0 selects greedy
    top_k: int = 0                # 0 disables the cut
    top_p: float = 1.0            # 1.0 disables it
    min_p: float = 0.0            # 0 disables it
    repeat_penalty: float = 1.0   # 1.0 disables it
    penalty_window: int = 64      # 0 means the whole history
    seed: int = 0                 # 0 selects the fixed default seed

    def validate(self) -> None:
        if math.isnan(self.temperature):
            raise ValueError("sampling: NaN temperature")
        if self.top_k < 0:
            raise ValueError("sampling: negative top_k")
        if math.isnan(self.top_p) or not 0.0 <= self.top_p <= 1.0:
            raise ValueError("sampling: top_p outside [0, 1]")
        if math.isnan(self.min_p) or not 0.0 <= self.min_p <= 1.0:
            raise ValueError("sampling: min_p outside [0, 1]")
        if not self.repeat_penalty > 0.0 or not math.isfinite(self.repeat_penalty):
            raise ValueError("sampling: repeat_penalty must be finite > 0")
        if self.penalty_window < 0:
            raise ValueError("sampling: negative penalty_window")
        if not 0 <= self.seed < 2 ** 32:
            raise ValueError("sampling: seed must fit 32 bits")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def has_cuts(self) -> bool:
        return self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0

    @property
    def has_penalty(self) -> bool:
        return self.repeat_penalty != 1.0


class XorShift32:
    """The reference's generator: one 32-bit word of state per request."""

    def __init__(self, seed: int = 0):
        self.state = (seed & 0xFFFFFFFF) or DEFAULT_SEED

    def next_uniform(self) -> float:
        """A float32-exact value in [0, 1): the top 24 bits of the new state over 2**24."""
        s = self.state
        if s == 0:
            s = DEFAULT_SEED
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        self.state = s
        return (s >> 8) / 16777216.0

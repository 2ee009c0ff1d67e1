"""Distributions of the random-weights mode and the key of a tensor (csrc/random_weights.h states the
arithmetic that turns a key and an element index into a value)."""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
NORMAL, UNIFORM = 0, 1


@dataclass(frozen=True)
class Draw:
    """How a tensor's elements are distributed; made by :func:`normal` or :func:`uniform`."""

    kind: int
    scale: float = 0.0      # normal: the factor of the integer sum
    base: int = 0           # uniform: lo * 2^24, rounded
    span: int = 0           # uniform: (hi - lo) * 2^24, rounded


def normal(std: float) -> Draw:
    """Mean 0, deviation ``std``: a centred sum of eight 16-bit uniform integers times a constant."""
    if not std > 0.0:
        raise ValueError("normal: the deviation must be positive")
    deviation_of_sum = 2.0 * math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)      # of 2 s - 8 * 65535
    return Draw(NORMAL, scale=ctypes.c_float(std / deviation_of_sum).value)


def uniform(lo: float, hi: float) -> Draw:
    """Uniform on [lo, hi) in steps of 2^-24."""
    base, span = round(lo * (1 << 24)), round((hi - lo) * (1 << 24))
    if not (0 < span < (1 << 31) and -(1 << 31) <= base and base + span < (1 << 31)):
        raise ValueError(f"uniform: [{lo}, {hi}) does not fit 32-bit fixed point with 24 fraction bits")
    return Draw(UNIFORM, base=base, span=span)


def _mix(z: int) -> int:
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor: FNV-1a of its name, mixed with the seed."""
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _MASK
    return _mix(h ^ _mix((int(seed) + _GOLDEN) & _MASK))

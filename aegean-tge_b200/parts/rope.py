"""Rotary position encoding, rotate-half ("NeoX") pairing.

As the reference builds it (src/models/qwen2.cpp:608-671): for pair index
``i < rotary/2`` the frequency is ``theta ** (-2i / rotary)`` evaluated in
float32, the angle of position ``p`` is ``float(p) * freq`` in float32, and
the tables hold ``cos`` and ``sin`` of that angle.  The rotation
(src/cpu/scalar/norm_rope_scalar.cpp:23-41) pairs element ``i`` with element
``i + rotary/2``:  ``lo' = lo*cos - hi*sin``, ``hi' = lo*sin + hi*cos``.
Values are not rotated, and keys are stored rotated.

The tables are computed on the host: the exponent and the angle in float32
exactly as above, ``pow``, ``cos`` and ``sin`` in float64 of those float32
arguments and rounded once, which is what a correctly rounded float32
routine returns.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import POSITIONS, PositionEncoding


def rotary_tables(theta: float, rotary: int, positions: int) -> Tuple[torch.Tensor, torch.Tensor]:
    half = rotary // 2
    index = torch.arange(half, dtype=torch.float32)
    exponent = (-2.0 * index) / torch.tensor(float(rotary), dtype=torch.float32)          # float32
    theta32 = torch.tensor(theta, dtype=torch.float32)
    freq = torch.pow(theta32.double(), exponent.double()).float()                           # rounded once
    angle = torch.arange(positions, dtype=torch.float32)[:, None] * freq[None, :]          # float32 product
    return torch.cos(angle.double()).float(), torch.sin(angle.double()).float()


_TABLES: dict = {}


@POSITIONS.register("rope_neox")
class RotaryNeoX(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default head_dim)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary <= 0 or self.rotary % 2 or self.rotary > self.head_dim:
            raise ValueError(f"rope: rotary width {self.rotary} must be even and within head_dim {self.head_dim}")
        if not self.theta > 0:
            raise ValueError("rope: theta must be positive")
        # layers with the same base, width and length share one pair of tables
        key = (self.theta, self.rotary, env.max_positions, str(env.device))
        if key not in _TABLES:
            if len(_TABLES) >= 8:
                _TABLES.pop(next(iter(_TABLES)))
            cos, sin = rotary_tables(self.theta, self.rotary, env.max_positions)
            _TABLES[key] = (cos.to(env.device).contiguous(), sin.to(env.device).contiguous())
        self.cos, self.sin = _TABLES[key]

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor, int]]:
        return self.cos, self.sin, self.rotary


@POSITIONS.register("none")
class NoPosition(PositionEncoding):
    """Leaves queries and keys as they are."""
    graph_safe = True

    def rotary_tables(self):
        return None, None, 0

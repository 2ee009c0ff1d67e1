"""RMSNorm with its epsilon as a parameter.

Formula of the reference (src/cpu/scalar/norm_rope_scalar.cpp:8-21): the sum
of squares in float32, ``scale = 1 / sqrt(sum / dim + eps)``, then
``x * scale * weight`` (scale first, weight second).  No bias, no ``+1`` on
the weight.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm, ParamSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size`` (row width), ``eps``.  weights: ``weight``."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        if self.size <= 0 or not self.eps > 0.0:
            raise ValueError(f"rmsnorm: size {self.size} and eps {self.eps} must be positive")
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector")}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.ops.rmsnorm(x, self.weight, self.eps, self.env.dtype, rows=rows)

    def fusable(self):
        return self.weight, self.eps

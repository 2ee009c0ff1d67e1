"""Dense gated feed-forward (SwiGLU).

Reference order (src/models/qwen2.cpp:2105-2118,
src/cpu/scalar/norm_rope_scalar.cpp:43-51): ``g = Wg h``, ``u = Wu h``,
``a_i = g_i / (1 + exp(-g_i)) * u_i``, ``d = Wd a``, added to the stream.  No
biases.  Gate and up rows are interleaved at load (row 2i = gate_i, row 2i+1
= up_i) so that one product yields both and its epilogue applies the gate.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import FEED_FORWARDS, FeedForward, ParamSpec, StepContext


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``.  weights: ``gate|up|down.weight``."""
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.inner = int(spec.params["intermediate_size"])
        if self.hidden <= 0 or self.inner <= 0:
            raise ValueError("swiglu: sizes must be positive")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate.weight": ParamSpec((self.inner, self.hidden)),
            "up.weight": ParamSpec((self.inner, self.hidden)),
            "down.weight": ParamSpec((self.hidden, self.inner)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        gate, up = tensors["gate.weight"], tensors["up.weight"]
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.inner, self.hidden).contiguous()
        self.w_down = tensors["down.weight"].contiguous()

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * 3 * self.inner * self.hidden

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        a = self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_SWIGLU)
        return self.ops.linear(a, self.w_down, None, self.ops.GEMM_STORE)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, next_norm=None, defer: bool = False):
        a = self.ops.linear(h, self.w_gate_up, None, self.ops.GEMM_SWIGLU)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_down, None, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_down, None, self.ops.GEMM_ADD_F32, out=x)
        return None

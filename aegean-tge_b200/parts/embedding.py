"""Token embedding and output head.

Embedding is a row copy with no scaling (src/models/qwen2.cpp:1143-1152,
:2050); the head is a plain product of the final-normed rows with the output
matrix, which is the embedding table itself when the model ties them
(src/models/qwen2.cpp:412-420, :2121-2122).  Logits are float32.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import EMBEDDINGS, HEADS, ParamSpec, Part


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: ``vocab_size``, ``hidden_size``.  weights: ``weight``."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def param_bytes(self) -> int:
        return 0        # a step reads the rows of its tokens, not the table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.ops.embedding(self.weight, token_ids)


@HEADS.register("linear_head")
class LinearHead(Part):
    """params: ``vocab_size``, ``hidden_size``.  weights: ``weight`` [vocab, hidden]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def flops(self, tokens: int, pairs: float) -> float:
        return 2.0 * tokens * self.vocab * self.hidden

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.ops.linear(h, self.weight, None, self.ops.GEMM_STORE_F32)

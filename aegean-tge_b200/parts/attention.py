"""Grouped-query attention over the paged cache.

In the reference's order (src/models/qwen2.cpp:2059-2103): three projections
of the normed input, then the biases, then the rotation of q and k, then the
cache write of rotated k and plain v, then for every query head ``h`` causal
softmax attention against kv head ``h // group`` with scores
``dot(q, k) * head_dim**-0.5`` (src/cpu/scalar/attention_scalar.cpp:48-115),
then the output projection added to the stream.  Here q, k and v are one
product over row-concatenated weights with the bias in its epilogue, the
rotation and the cache write are one kernel, and the output projection adds
into the float32 stream in its epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.model_spec import PartSpec
from .base import (MIXERS, POSITIONS, LayerCache, Mixer, PagedCacheSpec, ParamSpec, StepContext, build_part)


@MIXERS.register("gqa_attention")
class GQAttention(Mixer):
    """params: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``,
    ``qkv_bias`` (bool), ``o_bias`` (bool), ``window`` (None or tokens),
    ``position`` (a PartSpec), optional ``scale``.
    weights: ``q|k|v|o.weight`` and, with the bias flags, ``q|k|v|o.bias``.
    """
    graph_safe = True
    can_defer_norm = True
    takes_deferred_rows = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.o_bias = bool(p.get("o_bias", False))
        self.window = p.get("window")
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("attention: a window must be positive")
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        position: PartSpec = p.get("position", PartSpec("none"))
        self.position = build_part(POSITIONS, position, env)
        self.graph_safe = bool(self.position.graph_safe)
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.b_o: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {
            "q.weight": ParamSpec((self.q_dim, self.hidden)),
            "k.weight": ParamSpec((self.kv_dim, self.hidden)),
            "v.weight": ParamSpec((self.kv_dim, self.hidden)),
            "o.weight": ParamSpec((self.hidden, self.q_dim)),
        }
        if self.qkv_bias:
            specs["q.bias"] = ParamSpec((self.q_dim,), role="vector")
            specs["k.bias"] = ParamSpec((self.kv_dim,), role="vector")
            specs["v.bias"] = ParamSpec((self.kv_dim,), role="vector")
        if self.o_bias:
            specs["o.bias"] = ParamSpec((self.hidden,), role="vector")
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # rows of q, then k, then v: one product serves all three
        self.w_qkv = torch.cat([tensors["q.weight"], tensors["k.weight"], tensors["v.weight"]], dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q.bias"], tensors["k.bias"], tensors["v.bias"]]).contiguous()
        self.w_o = tensors["o.weight"].contiguous()
        self.b_o = tensors["o.bias"].contiguous() if self.o_bias else None

    def flops(self, tokens: int, pairs: float) -> float:
        products = 2.0 * tokens * (self.q_dim + 2 * self.kv_dim + self.q_dim) * self.hidden
        return products + 4.0 * self.heads * self.head_dim * pairs         # scores and weighted values

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        entry = (self.kv_heads, self.head_dim)
        return PagedCacheSpec(entries=(("k", entry), ("v", entry)),
                              window=None if self.window is None else int(self.window))

    def attend(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """Everything up to, not including, the output projection: [T, heads*head_dim]."""
        ops = self.ops
        k_pages, v_pages = cache.paged["k"], cache.paged["v"]
        table = ctx.block_tables[cache.group]
        tables = self.position.rotary_tables()
        if tables is not None and cache.owner:
            # product, bias, rotation and cache store together (one or two kernels, chosen by batch size)
            cos, sin, rotary = tables
            qkv = ops.linear_qkv_rope_store(h, self.w_qkv, self.b_qkv, cos, sin, rotary, ctx.positions,
                                            ctx.seq_of_token, table, k_pages, v_pages, self.heads, self.kv_heads,
                                            self.head_dim)
        else:
            qkv = ops.linear(h, self.w_qkv, self.b_qkv, ops.GEMM_STORE)
            if tables is None:
                q = qkv[:, :self.q_dim].view(-1, self.heads, self.head_dim)
                k = qkv[:, self.q_dim:self.q_dim + self.kv_dim].view(-1, self.kv_heads, self.head_dim)
                self.position.apply(q, k, ctx.positions)
                cos = sin = None
                rotary = 0
            else:
                cos, sin, rotary = tables
            ops.rope_kv_store(qkv, cos, sin, rotary, ctx.positions, ctx.seq_of_token, table,
                              k_pages if cache.owner else None, v_pages if cache.owner else None,
                              self.heads, self.kv_heads, self.head_dim)
        return ops.attention(qkv[:, :self.q_dim], k_pages, v_pages, table, ctx.q_start, ctx.start_pos, ctx.positions,
                             ctx.seq_of_token, ctx.num_seqs, ctx.max_q_len, ctx.max_ctx_len, self.heads,
                             self.kv_heads, self.head_dim, self.scale, window=int(self.window or 0),
                             split_tokens=ctx.attn_split_tokens, typical_ctx_len=ctx.typical_ctx_len,
                             decode_prefix=ctx.decode_prefix)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        return self.ops.linear(self.attend(h, ctx, cache), self.w_o, self.b_o, self.ops.GEMM_STORE)

    def forward_add(self, h: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: LayerCache, next_norm=None,
                    defer: bool = False):
        a = self.attend(h, ctx, cache)
        fused = next_norm.fusable() if next_norm is not None else None
        if fused is not None:
            return self.ops.linear_add_norm(a, self.w_o, self.b_o, x, fused[0], fused[1], self.env.dtype, defer=defer)
        self.ops.linear(a, self.w_o, self.b_o, self.ops.GEMM_ADD_F32, out=x)
        return None

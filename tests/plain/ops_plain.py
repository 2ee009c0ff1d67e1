"""Plain float64 references of single kernels, for the per-kernel tests.

Each function restates one formula of the reference (cited) on whole tensors,
with no tiling, no pages beyond a gather, and no code shared with the package.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

F = torch.float64


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/cpu/scalar/norm_rope_scalar.cpp:8-21"""
    x = x.to(F)
    s = (x * x).sum(-1, keepdim=True)
    return x * (1.0 / torch.sqrt(s / x.shape[-1] + eps)) * weight.to(F)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Row-times-vector products (src/tensor/reference.cpp:29-45), bias after the product
    (src/models/qwen2.cpp:2062-2068)."""
    y = x.to(F) @ w.to(F).T
    return y if bias is None else y + bias.to(F)


def swiglu_interleaved(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """Rows 2i / 2i+1 of the weight are gate_i / up_i; a_i = g/(1+exp(-g))*u
    (src/cpu/scalar/norm_rope_scalar.cpp:43-51)."""
    y = x.to(F) @ w_gate_up.to(F).T
    g, u = y[:, 0::2], y[:, 1::2]
    return g / (1.0 + torch.exp(-g)) * u


def rotate_half(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary: int) -> torch.Tensor:
    """v [T, heads, hd], cos/sin [T, rotary/2] (src/cpu/scalar/norm_rope_scalar.cpp:23-41);
    dimensions beyond ``rotary`` pass through."""
    v = v.to(F)
    half = rotary // 2
    if half == 0:
        return v
    lo, hi, rest = v[..., :half], v[..., half:rotary], v[..., rotary:]
    c, s = cos.to(F)[:, None, :], sin.to(F)[:, None, :]
    return torch.cat([lo * c - hi * s, lo * s + hi * c, rest], dim=-1)


def gather_pages(pages: torch.Tensor, table_row, length: int) -> torch.Tensor:
    """pages [num_pages, kv_heads, page, hd] -> contiguous [length, kv_heads, hd] of one request."""
    page_size = pages.shape[2]
    rows = []
    for pos in range(length):
        rows.append(pages[int(table_row[pos // page_size]), :, pos % page_size, :])
    return torch.stack(rows).to(F)


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions, scale: float,
                   window: int = 0) -> torch.Tensor:
    """q [n, heads, hd] at absolute ``positions`` against one request's k/v [ctx, kv_heads, hd]
    (src/cpu/scalar/attention_scalar.cpp:48-115): keys 0..p, scale after the dot, softmax, mix."""
    n, heads, hd = q.shape
    group = heads // k.shape[1]
    q, k, v = q.to(F), k.to(F), v.to(F)
    out = torch.zeros(n, heads, hd, dtype=F)
    for i in range(n):
        p = int(positions[i])
        first = max(p - window + 1, 0) if window > 0 else 0
        for h in range(heads):
            s = (k[first:p + 1, h // group] @ q[i, h]) * scale
            e = torch.exp(s - s.max())
            out[i, h] = (e / e.sum()) @ v[first:p + 1, h // group]
    return out

"""A plain, slow implementation of the Qwen2.5 dense decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function per part, float64
arithmetic on the CPU.  It shares no code with the package: it reads
config.json and the safetensors file with the `safetensors` library and
restates the reference's formulas, each cited by file:line of the reference
(paths within AegeanWorks/Aegean-TGE).

It rests on the reference in two ways: on its formulas (cited below), and on a
one-time comparison of this file with the reference's own model code compiled
on the CPU, whose inputs and outputs are kept under tests/golden/ (see
tests/golden/make_golden.py and tests/test_plain_vs_golden.py).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Sequence

import numpy as np
import torch
from safetensors import safe_open

F = torch.float64


def read_model(model_dir: str):
    """(config dict, {tensor name: float64 tensor})."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        config = json.load(handle)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(F)
    return config, weights


def sizes(config: dict):
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads") or heads          # qwen2.cpp:235-238
    head_dim = config.get("head_dim") or config["hidden_size"] // heads   # qwen2.cpp:342-344
    return heads, kv_heads, head_dim


def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[t] = E[token_t]: a row copy, no scaling (src/models/qwen2.cpp:1143-1152, :2050)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].clone()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """s = sum x^2; scale = 1/sqrt(s/dim + eps); out = x*scale*w (src/cpu/scalar/norm_rope_scalar.cpp:8-21)."""
    s = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(s / x.shape[-1] + eps)
    return x * scale * weight


def rope_tables(theta: float, head_dim: int, positions: int):
    """cos/sin tables as the loader builds them (src/models/qwen2.cpp:608-617, :657-671).

    The reference evaluates the exponent, the power and the angle in float32:
    freq_i = powf(theta, -2.0f*i/head_dim), angle = float(p) * freq_i.  The same
    float32 values are formed here (the power via float64 and one rounding), and
    the cosine and sine of that float32 angle are taken in float64.
    """
    half = head_dim // 2
    exponent = (np.float32(-2.0) * np.arange(half, dtype=np.float32)) / np.float32(head_dim)
    freq = np.power(np.float64(np.float32(theta)), exponent.astype(np.float64)).astype(np.float32)
    angle = np.arange(positions, dtype=np.float32)[:, None] * freq[None, :]
    angle = angle.astype(np.float64)
    return torch.from_numpy(np.cos(angle)), torch.from_numpy(np.sin(angle))


def apply_rope(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing on [T, heads, head_dim] (src/cpu/scalar/norm_rope_scalar.cpp:23-41):
    lo' = lo*c - hi*s ; hi' = lo*s + hi*c with lo = v[i], hi = v[i + head_dim/2]."""
    half = v.shape[-1] // 2
    lo, hi = v[..., :half], v[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, lo * s + hi * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0) -> torch.Tensor:
    """Causal softmax attention, one query head at a time (src/cpu/scalar/attention_scalar.cpp:48-115,
    src/models/qwen2.cpp:1243-1304).  q [T, heads, hd], k/v [T, kv_heads, hd].

    kv head = h // group (qwen2.cpp:1248-1249); for the row at position p the keys are
    t = 0..p (the causal mask is the loop bound, qwen2.cpp:1276); s_t = dot * scale with
    scale = 1/sqrt(hd) applied after the dot (attention_scalar.cpp:66-80); m = max s;
    e = exp(s - m); w = e / sum e; out = sum w_t v_t (attention_scalar.cpp:84-114).
    ``window`` > 0 keeps only the last ``window`` keys (not part of the reference).
    """
    T, heads, hd = q.shape
    group = heads // k.shape[1]
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    for h in range(heads):
        kh = h // group
        for p in range(T):
            first = max(p - window + 1, 0) if window > 0 else 0
            s = (k[first:p + 1, kh] @ q[p, h]) * scale
            e = torch.exp(s - s.max())
            w = e / e.sum()
            out[p, h] = w @ v[first:p + 1, kh]
    return out


def swiglu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """g = Wg h; u = Wu h; a = g/(1+exp(-g))*u; d = Wd a (src/models/qwen2.cpp:2105-2118,
    src/cpu/scalar/norm_rope_scalar.cpp:43-51)."""
    g = h @ gate.T
    u = h @ up.T
    a = g / (1.0 + torch.exp(-g)) * u
    return a @ down.T


def layer(x: torch.Tensor, n: int, config: dict, w: Dict[str, torch.Tensor], cos, sin) -> torch.Tensor:
    """One decoder layer in the reference's order (src/models/qwen2.cpp:2055-2118): norm, q/k/v products,
    then the biases (:2062-2068), rotation of q and k (:2070-2072), attention, output product without
    bias added to the stream (:2099-2103), norm, feed-forward added to the stream."""
    heads, kv_heads, hd = sizes(config)
    eps = config.get("rms_norm_eps", 1e-6)
    p = f"model.layers.{n}."
    T = x.shape[0]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = h @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]
    k = h @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]
    v = h @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]
    q = apply_rope(q.view(T, heads, hd), cos[:T], sin[:T])
    k = apply_rope(k.view(T, kv_heads, hd), cos[:T], sin[:T])
    a = attention(q, k, v.view(T, kv_heads, hd)).reshape(T, heads * hd)
    x = x + a @ w[p + "self_attn.o_proj.weight"].T
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
    return x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def logits_of(config: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  Final norm and head as src/models/qwen2.cpp:2121-2122;
    the head is the embedding table when the file has no output matrix (:412-420)."""
    _, _, hd = sizes(config)
    cos, sin = rope_tables(config.get("rope_theta", 10000.0), hd, len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens)
    for n in range(config["num_hidden_layers"]):
        x = layer(x, n, config, w, cos, sin)
    h = rms_norm(x, w["model.norm.weight"], config.get("rms_norm_eps", 1e-6))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return h @ head.T


def greedy(config: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n: int) -> List[int]:
    """Greedy continuation by recomputing the whole sequence each time; first maximal index
    (src/models/sampling.cpp:198-207)."""
    tokens = list(prompt)
    out: List[int] = []
    for _ in range(n):
        row = logits_of(config, w, tokens)[-1].to(torch.float32)
        token = int(torch.argmax(row))      # torch returns the first maximal index
        out.append(token)
        tokens.append(token)
    return out


# ---------------------------------------------------------------------------
# sampler (src/models/sampling.cpp:16-28, :72-93, :183-228; norm_rope_scalar.cpp:53-72)
# ---------------------------------------------------------------------------
class PlainXorShift32:
    def __init__(self, seed: int):
        self.state = (seed & 0xFFFFFFFF) or 0x9E3779B9

    def next(self) -> np.float32:
        s = self.state
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        self.state = s
        return np.float32(s >> 8) / np.float32(16777216.0)


def sample_plain(logits: np.ndarray, temperature: float, rng: PlainXorShift32) -> int:
    """Greedy (first maximum) or a temperature draw by the sequential float32 walk."""
    logits = logits.astype(np.float32)
    if temperature <= 0.0:
        best = 0
        for i in range(1, len(logits)):
            if logits[i] > logits[best]:
                best = i
        return best
    inv = np.float32(1.0) / np.float32(temperature)
    e = np.exp((logits - logits.max()) * inv).astype(np.float32)
    total = np.float32(0.0)
    for value in e:
        total = np.float32(total + value)
    if not total > 0:
        return 0
    target = np.float32(rng.next() * total)
    for i, value in enumerate(e):
        target = np.float32(target - value)
        if target <= 0:
            return i
    return len(e) - 1


def penalize_plain(logits: np.ndarray, history: Sequence[int], penalty: float, window: int) -> np.ndarray:
    """Repetition penalty (src/models/sampling.cpp:32-54): each distinct token of the last ``window``
    history tokens (0 = all) once; positive scores are divided, negative ones multiplied."""
    scores = logits.astype(np.float32).copy()
    if not (penalty > 0.0 and penalty != 1.0 and len(history) > 0):
        return scores
    begin = max(0, len(history) - window) if window > 0 else 0
    seen = set()
    for token in reversed(history[begin:]):
        if token < 0 or token >= len(scores) or token in seen:
            continue
        seen.add(token)
        scores[token] = scores[token] / np.float32(penalty) if scores[token] > 0 else scores[token] * np.float32(penalty)
    return scores


def sample_cuts_plain(scores: np.ndarray, temperature: float, top_k: int, top_p: float, min_p: float, u: float) -> int:
    """Temperature draw with the top-k / min-p / top-p cuts (src/models/sampling.cpp:230-410), float32,
    sequential.  Candidates are ordered by probability, highest first, lower index first among equals."""
    scores = scores.astype(np.float32)
    count = len(scores)
    inv = np.float32(1.0) / np.float32(temperature)
    prob = np.exp((scores - scores.max()) * inv).astype(np.float32)
    order = sorted(range(count), key=lambda i: (-float(prob[i]), i))
    keep = min(top_k, count) if top_k > 0 else count
    order = order[:keep]
    if min_p > 0.0:
        floor = np.float32(min_p) * prob[order[0]]
        order = [i for i in order if prob[i] >= floor]
    total = np.float32(0.0)
    for i in order:
        total = np.float32(total + prob[i])
    if not order or not total > 0:
        return int(np.argmax(prob))
    limit = len(order)
    if top_p < 1.0:
        cumulative = np.float32(0.0)
        for n, i in enumerate(order):
            cumulative = np.float32(cumulative + prob[i])
            if cumulative / total >= np.float32(top_p):
                limit = n + 1
                break
    kept = np.float32(0.0)
    for i in order[:limit]:
        kept = np.float32(kept + prob[i])
    target = np.float32(np.float32(u) * kept)
    for i in order[:limit]:
        target = np.float32(target - prob[i])
        if target <= 0:
            return i
    return order[limit - 1]

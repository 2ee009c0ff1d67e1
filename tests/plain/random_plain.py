"""The engine's random weights, restated with numpy: the tests' own source of a seeded model.

It shares no code with the package.  The rule (the package states it in csrc/random_weights.h): an
element of a tensor is a function of the seed, the tensor's name and the element's row-major index,

    mix(z)    : z ^= z >> 30; z *= 0xBF58476D1CE4E5B9; z ^= z >> 27; z *= 0x94D049BB133111EB; z ^= z >> 31
    key       : mix(fnv1a64(name) ^ mix(seed + 0x9E3779B97F4A7C15))
    word(c)   : mix(key + 0x9E3779B97F4A7C15 * (c + 1))
    normal i  : s = the eight 16-bit fields of word(2i) and word(2i+1) added up;
                value = float32(2 s - 8 * 65535) * float32(std / (2 sqrt(8 (65536^2 - 1) / 12)))
    uniform i : m = round(lo 2^24) + ((word(i) >> 32) * round((hi - lo) 2^24) >> 32); value = float32(m) * 2^-24

all integer arithmetic modulo 2^64, the last step one correctly rounded float32 multiplication.
"""
from __future__ import annotations

import math
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterator, Sequence, Tuple

import numpy as np

U = np.uint64
GOLDEN = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1


def _mix_int(z: int) -> int:
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def key_of(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & MASK
    return _mix_int(h ^ _mix_int((seed + GOLDEN) & MASK))


CHUNK = 1 << 15      # elements per piece: its work arrays stay in the cache
THREADS = min(8, os.cpu_count() or 1)


def _words(key: int, z: np.ndarray, t: np.ndarray) -> None:
    """z holds counters on entry and their words on return (t is work space)."""
    with np.errstate(over="ignore"):
        z += U(1)
        z *= U(GOLDEN)
        z += U(key)
        for shift, factor in ((30, 0xBF58476D1CE4E5B9), (27, 0x94D049BB133111EB)):
            np.right_shift(z, U(shift), out=t)
            z ^= t
            z *= U(factor)
        np.right_shift(z, U(31), out=t)
        z ^= t


def _fields(z: np.ndarray, t: np.ndarray) -> None:
    """z becomes the sum of its four 16-bit fields."""
    np.right_shift(z, U(16), out=t)
    t &= U(0x0000FFFF0000FFFF)
    z &= U(0x0000FFFF0000FFFF)
    z += t                                  # two sums of two fields, in the two halves
    np.right_shift(z, U(32), out=t)
    z &= U(0xFFFFFFFF)
    z += t


class _Work:
    """Work arrays of one thread, used again for every piece it computes."""

    def __init__(self):
        self.a, self.b, self.t = (np.empty(CHUNK, dtype=U) for _ in range(3))
        self.i = np.empty(CHUNK, dtype=np.int64)
        self.f = np.empty(CHUNK, dtype=np.float32)


def _normal_piece(key: int, first: int, out: np.ndarray, scale: np.float32, work: _Work) -> None:
    n = out.size
    a, b, t, centred, f = work.a[:n], work.b[:n], work.t[:n], work.i[:n], work.f[:n]
    a[:] = np.arange(first, first + n, dtype=U)
    a *= U(2)
    np.add(a, U(1), out=b)
    for z in (a, b):
        _words(key, z, t)
        _fields(z, t)
    a += b
    centred[:] = a
    centred *= 2
    centred -= 8 * 65535
    f[:] = centred                          # exact: the magnitude stays below 2^20
    np.multiply(f, scale, out=out)


def _uniform_piece(key: int, first: int, out: np.ndarray, base: int, span: int, work: _Work) -> None:
    n = out.size
    z, t, m, f = work.a[:n], work.t[:n], work.i[:n], work.f[:n]
    z[:] = np.arange(first, first + n, dtype=U)
    _words(key, z, t)
    z >>= U(32)
    z *= U(span)
    z >>= U(32)
    m[:] = z
    m += base
    f[:] = m                                # rounds to nearest even above 2^24, as the engine's conversion does
    np.multiply(f, np.float32(2.0 ** -24), out=out)


def tensor(seed: int, name: str, shape: Sequence[int], draw: Tuple, first: int = 0, count: int = -1) -> np.ndarray:
    """float32 tensor ``name`` of the model with this seed.  ``draw``: ("normal", std) or ("uniform", lo, hi).
    ``first``/``count`` pick a run of the flattened tensor instead of all of it."""
    whole = count < 0
    if whole:
        first, count = 0, int(np.prod(shape))
    key = key_of(seed, name)
    flat = np.empty(count, dtype=np.float32)
    if draw[0] == "normal":
        scale = np.float32(draw[1] / (2.0 * math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)))

        def piece(begin, work):
            _normal_piece(key, first + begin, flat[begin:begin + CHUNK], scale, work)
    else:
        base, span = round(draw[1] * (1 << 24)), round((draw[2] - draw[1]) * (1 << 24))

        def piece(begin, work):
            _uniform_piece(key, first + begin, flat[begin:begin + CHUNK], base, span, work)

    def span_of_pieces(begins):
        work = _Work()
        for begin in begins:
            piece(begin, work)
    begins = list(range(0, count, CHUNK))
    workers = min(THREADS, len(begins) // 16)
    if workers > 1:
        share = -(-len(begins) // workers)
        with ThreadPoolExecutor(max_workers=workers) as pool:
            list(pool.map(span_of_pieces, [begins[w * share:(w + 1) * share] for w in range(workers)]))
    else:
        span_of_pieces(begins)
    return flat.reshape(shape) if whole else flat


def to_bfloat16(x: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), still stored as float32."""
    bits = x.astype(np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def qwen2_plan(config: dict) -> Iterator[Tuple[str, Tuple[int, ...], str, Tuple]]:
    """(name, shape, role, draw) of a Qwen2.5 checkpoint: matrices and biases N(0, 0.02), norm weights
    1 + U(-0.1, 0.1) (what the engine's random-weights mode draws for this architecture)."""
    h, ff, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    heads = config["num_attention_heads"]
    kv_heads = config.get("num_key_value_heads") or heads
    hd = config.get("head_dim") or h // heads
    q, kv = heads * hd, kv_heads * hd
    n02, norm = ("normal", 0.02), ("uniform", 0.9, 1.1)
    yield "model.embed_tokens.weight", (v, h), "matrix", n02
    for n in range(config["num_hidden_layers"]):
        p = f"model.layers.{n}."
        yield p + "input_layernorm.weight", (h,), "vector", norm
        for x, rows in (("q", q), ("k", kv), ("v", kv)):
            yield p + f"self_attn.{x}_proj.weight", (rows, h), "matrix", n02
            yield p + f"self_attn.{x}_proj.bias", (rows,), "vector", n02
        yield p + "self_attn.o_proj.weight", (h, q), "matrix", n02
        yield p + "post_attention_layernorm.weight", (h,), "vector", norm
        yield p + "mlp.gate_proj.weight", (ff, h), "matrix", n02
        yield p + "mlp.up_proj.weight", (ff, h), "matrix", n02
        yield p + "mlp.down_proj.weight", (h, ff), "matrix", n02
    yield "model.norm.weight", (h,), "vector", norm
    if not config.get("tie_word_embeddings", False):
        yield "lm_head.weight", (v, h), "matrix", n02


def qwen2_weights(config: dict, seed: int, matrices_as_bfloat16: bool = False) -> Dict[str, np.ndarray]:
    """All tensors of the model as float32 arrays; matrices optionally rounded to bfloat16 values."""
    out = {}
    for name, shape, role, draw in qwen2_plan(config):
        value = tensor(seed, name, shape, draw)
        out[name] = to_bfloat16(value) if matrices_as_bfloat16 and role == "matrix" else value
    return out

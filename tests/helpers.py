"""Helpers shared by the GPU tests."""
import random

import torch


def rel_error(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference over the largest reference magnitude."""
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), "non-finite values in the result"
    scale = max(float(ref.abs().max()), 1e-30)
    return float((got - ref).abs().max()) / scale


# Tolerances, fixed once: float32 kernels differ from float64 by summation rounding;
# bfloat16 results carry one rounding of the output (2^-9) plus rounded intermediates.
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}
# Whole-model logits against the float64 plain model with float32 weights, relative to the largest logit:
# about three times the largest error seen on a B200 (float32 2.4e-6 with the toy parts, 9e-7 otherwise;
# bfloat16 1.1e-2 with the toy parts).  Per tiny configuration the bfloat16 bound is tighter: model_tol().
MODEL_TOL = {"float32": 1e-5, "bfloat16": 3.5e-2}
# largest bfloat16 error seen: A 3.1e-3, B 7.8e-3, C 7.0e-3, D 8.8e-3, E 4.1e-3
_BFLOAT16_TOL = {"A": 1e-2, "B": 2.5e-2, "C": 2.2e-2, "D": 2.7e-2, "E": 1.3e-2}


def model_tol(dtype: str, name: str = "") -> float:
    """The bound for whole-model logits of tiny configuration ``name`` (the general bound if it has none)."""
    if dtype == "bfloat16":
        return _BFLOAT16_TOL.get(name, MODEL_TOL[dtype])
    return MODEL_TOL[dtype]


def paged_cache(lengths, kv_heads, head_dim, page_size, dtype, device, seed=0, extra_pages=3):
    """Random keys/values for requests of the given lengths, scattered over shuffled pages.

    Returns (k_pages, v_pages, block_table [S, W] int32, k_list, v_list) where k_list[s] is the
    contiguous [len, kv_heads, hd] tensor (already rounded to ``dtype``) of request s.
    """
    gen = torch.Generator().manual_seed(seed)
    need = [-(-n // page_size) for n in lengths]
    num_pages = sum(need) + extra_pages
    order = list(range(num_pages))
    random.Random(seed).shuffle(order)
    k_pages = torch.randn(num_pages, kv_heads, page_size, head_dim, generator=gen).to(dtype)   # stale junk, finite
    v_pages = torch.randn(num_pages, kv_heads, page_size, head_dim, generator=gen).to(dtype)
    width = max(need)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    k_list, v_list = [], []
    cursor = 0
    for s, n in enumerate(lengths):
        k = torch.randn(n, kv_heads, head_dim, generator=gen).to(dtype)
        v = torch.randn(n, kv_heads, head_dim, generator=gen).to(dtype)
        for j in range(need[s]):
            page = order[cursor]
            cursor += 1
            table[s, j] = page
            lo, hi = j * page_size, min((j + 1) * page_size, n)
            k_pages[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_pages[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        k_list.append(k)
        v_list.append(v)
    return k_pages.to(device), v_pages.to(device), table.to(device), k_list, v_list


def batch_index(q_lens, start_positions, device):
    """The int32 index tensors of a step made of portions with the given lengths and start positions."""
    positions, seq_of_token, q_start = [], [], [0]
    for s, (n, start) in enumerate(zip(q_lens, start_positions)):
        positions += list(range(start, start + n))
        seq_of_token += [s] * n
        q_start.append(q_start[-1] + n)
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return mk(positions), mk(seq_of_token), mk(q_start), mk(list(start_positions))

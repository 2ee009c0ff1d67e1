"""Random-weights mode: a model folder, or a model on the device, from a configuration and a seed.

The reference has no random model (its fixture is all zeros,
tests/test_gguf.cpp:962-1018, and its benches draw from an LCG,
apps/cli/main.cpp:154-161), so the generator is this engine's own.  It is
counter-based: an element's value is a function of the seed, the tensor's
checkpoint name and the element's row-major index and of nothing else
(csrc/random_weights.h states the arithmetic).  The same seed therefore gives
the same model whether it is drawn by the kernel on the device
(:func:`fill_random`, a 32B model in seconds, never on disk), by the host loop
behind ``tge make-random`` (:func:`write_random_model`), or by an independent
restatement such as the one the tests keep beside their plain model.

An architecture says which tensors exist and how each is distributed through
its ``random_plan``: ``(name, shape, role, draw)`` with ``draw`` one of
:func:`normal` and :func:`uniform`; role "matrix" is stored in the asked dtype,
role "vector" in float32.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Iterator, Sequence, Tuple

import torch

from ..registry import architecture_of
from .draws import Draw, normal, tensor_key, uniform  # noqa: F401  (re-exported)
from .loader import load_tensors, write_model_folder

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name: str) -> torch.dtype:
    if name not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{name}'")
    return _DTYPES[name]


def random_tensor(name: str, shape: Sequence[int], draw: Draw, seed: int, dtype: torch.dtype,
                  device: torch.device) -> torch.Tensor:
    """The tensor ``name`` of the model with this seed, drawn where it is wanted (kernel or host loop)."""
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"random weights are float32 or bfloat16, not {dtype}")
    device = torch.device(device)
    out = torch.empty(tuple(int(s) for s in shape), dtype=dtype, device=device)
    key = tensor_key(seed, name)
    is_bf16 = int(dtype == torch.bfloat16)
    if device.type == "cuda":
        from .. import ops
        with torch.cuda.device(device):
            lib = ops.core()
            ops._check(lib.tge_random_fill(out.data_ptr(), is_bf16, out.numel(), 0, key, draw.kind, draw.scale,
                                           draw.base, draw.span, ops._stream()), lib)
    else:
        from .. import runtime
        runtime.check(runtime.lib().tge_rt_random_fill(out.data_ptr(), is_bf16, out.numel(), 0, key, draw.kind,
                                                       draw.scale, draw.base, draw.span, os.cpu_count() or 1))
    return out


def random_tensors(raw_config: Dict[str, Any], seed: int, matrix_dtype: torch.dtype,
                   device: torch.device) -> Iterator[Tuple[str, torch.Tensor]]:
    """Every checkpoint tensor of the architecture ``raw_config`` names, one at a time."""
    arch = architecture_of(raw_config)
    config = arch.parse_config(raw_config)
    for name, shape, role, draw in arch.random_plan(config):
        if role not in ("matrix", "vector"):
            raise ValueError(f"random plan: tensor '{name}' has role '{role}', expected matrix or vector")
        yield name, random_tensor(name, shape, draw, seed, matrix_dtype if role == "matrix" else torch.float32, device)


def write_random_model(out_dir: str, raw_config: Dict[str, Any], seed: int, dtype: str = "float32") -> None:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` with seeded random weights.

    ``dtype`` is how matrices are stored (biases and norm weights are always float32).
    """
    stored = dict(raw_config)
    stored["torch_dtype"] = "float32" if parse_dtype(dtype) == torch.float32 else "bfloat16"
    write_model_folder(out_dir, stored, random_tensors(raw_config, seed, parse_dtype(dtype), torch.device("cpu")))


def fill_random(model, raw_config: Dict[str, Any], seed: int) -> None:
    """Seeded random weights drawn on the model's own device: the model ``write_random_model`` writes."""
    load_tensors(model, random_tensors(raw_config, seed, model.env.dtype, model.env.device))

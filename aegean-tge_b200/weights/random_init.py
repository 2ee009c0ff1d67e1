"""Random-weights mode: a model folder from a configuration and a seed.

The reference has no random model (its fixture is all zeros,
tests/test_gguf.cpp:962-1018, and its benches draw from an LCG,
apps/cli/main.cpp:154-161).  Here the architecture's ``random_tensors`` draws
matrices and biases from N(0, 0.02) and norm weights from 1 + U(-0.1, 0.1)
with a seeded generator; the result is written as a model folder or handed
straight to a model on the device (a 7B model then never touches the disk).
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..registry import architecture_of
from .loader import load_tensors, write_model_folder

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_dtype(name: str) -> torch.dtype:
    if name not in _DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{name}'")
    return _DTYPES[name]


def write_random_model(out_dir: str, raw_config: Dict[str, Any], seed: int, dtype: str = "float32") -> None:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors`` with seeded random weights.

    ``dtype`` is how matrices are stored (biases and norm weights are always float32).
    """
    arch = architecture_of(raw_config)
    config = arch.parse_config(raw_config)
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    stored = dict(raw_config)
    stored["torch_dtype"] = "float32" if parse_dtype(dtype) == torch.float32 else "bfloat16"
    write_model_folder(out_dir, stored,
                       arch.random_tensors(config, generator, parse_dtype(dtype), torch.device("cpu")))


def fill_random(model, raw_config: Dict[str, Any], seed: int) -> None:
    """Seeded random weights drawn on the model's own device."""
    arch = architecture_of(raw_config)
    config = arch.parse_config(raw_config)
    device = model.env.device
    generator = torch.Generator(device=device)
    generator.manual_seed(int(seed))
    load_tensors(model, arch.random_tensors(config, generator, model.env.dtype, device))

"""Binding checkpoint tensors to a model by name, with one error for everything wrong.

The reference finds every tensor by name and checks type, rank and shape
before it takes a view (src/models/qwen2.cpp:833-933), failing on the first
problem.  Here all problems are collected first: tensors the model wants and
the file lacks, tensors the file holds and the model does not want, and
tensors of the wrong shape or of a non-numeric type are listed together in a
single :class:`WeightError`.

What dtype a tensor has on the device depends on its role (``ParamSpec.role``)
and the run dtype:

* matrix (product operands, embedding table): the run dtype - bfloat16 in the
  serving path, float32 in the 32-bit path;
* vector (norm weights, biases): float32 always; a vector stored in 32-bit
  stays as it is and one stored in 16-bit is widened, which is exact;
* table (integers): int32.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import ModelFiles, write_safetensors

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(RuntimeError):
    """The checkpoint does not match the model.  ``missing``, ``unexpected`` and ``mismatched`` say how."""

    def __init__(self, missing: List[str], unexpected: List[str], mismatched: List[str]):
        self.missing, self.unexpected, self.mismatched = missing, unexpected, mismatched
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if mismatched:
            lines.append(f"  wrong shape or type ({len(mismatched)}): " + "; ".join(mismatched))
        super().__init__("\n".join(lines))


def device_dtype(param: ParamSpec, run_dtype: torch.dtype) -> torch.dtype:
    if param.role == "matrix":
        return run_dtype
    if param.role == "vector":
        return torch.float32
    if param.role == "table":
        return torch.int32
    raise ValueError(f"unknown parameter role '{param.role}'")


def check_against_manifest(entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]],
                           manifest: Dict[str, Tuple[ParamSpec, str]]) -> None:
    """``entries``: tensor name -> (stored dtype, shape).  Raises one WeightError for every problem."""
    missing = sorted(name for name, (param, _) in manifest.items() if name not in entries and not param.optional)
    unexpected = sorted(name for name in entries if name not in manifest)
    mismatched = []
    for name, (param, where) in sorted(manifest.items()):
        if name not in entries:
            continue
        dtype, shape = entries[name]
        if tuple(shape) != tuple(param.shape):
            mismatched.append(f"{name}: file has shape {list(shape)}, {where} needs {list(param.shape)}")
        elif param.role == "table" and dtype not in _INTS:
            mismatched.append(f"{name}: file has {dtype}, {where} needs integers")
        elif param.role != "table" and dtype not in _FLOATS:
            mismatched.append(f"{name}: file has {dtype}, {where} needs a floating type")
    if missing or unexpected or mismatched:
        raise WeightError(missing, unexpected, mismatched)


class Uploader:
    """Moves tensors from the mapped file to the device through a ring of pinned buffers.

    A plain ``tensor.to(device)`` from a mapped file faults its pages in one thread and copies from pageable
    memory: 2.3 GB/s with the file in the page cache.  Here a few threads copy slices of the file into pinned
    buffers (the page faults then run side by side), each buffer goes to the device asynchronously and is cast
    there to the dtype the model wants, and the next buffer is filled meanwhile.
    """

    CHUNK_BYTES = 64 << 20
    RING = 3
    THREADS = 4

    def __init__(self, device: torch.device):
        from concurrent.futures import ThreadPoolExecutor
        self.device = device
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.buffers = [torch.empty(self.CHUNK_BYTES, dtype=torch.uint8).pin_memory() for _ in range(self.RING)]
            self.free_again = [None] * self.RING         # the event after which a buffer may be overwritten
            self.pool = ThreadPoolExecutor(self.THREADS)
            self.turn = 0

    def upload(self, host: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        if not self.cuda or host.numel() * host.element_size() < (1 << 20):
            return host.to(device=self.device, dtype=dtype).contiguous()
        out = torch.empty(host.shape, dtype=dtype, device=self.device)
        flat_in, flat_out = host.reshape(-1), out.view(-1)
        per_chunk = self.CHUNK_BYTES // host.element_size()
        for first in range(0, flat_in.numel(), per_chunk):
            count = min(per_chunk, flat_in.numel() - first)
            turn = self.turn
            self.turn = (turn + 1) % self.RING
            if self.free_again[turn] is not None:
                self.free_again[turn].synchronize()
            staged = self.buffers[turn].view(host.dtype)[:count]
            piece = -(-count // self.THREADS)
            jobs = [self.pool.submit(staged[i:i + piece].copy_, flat_in[first + i:first + i + piece])
                    for i in range(0, count, piece)]
            for job in jobs:
                job.result()
            if host.dtype == dtype:
                flat_out[first:first + count].copy_(staged, non_blocking=True)
            else:                                        # as stored to the device, cast there
                arrived = torch.empty(count, dtype=host.dtype, device=self.device)
                arrived.copy_(staged, non_blocking=True)
                flat_out[first:first + count].copy_(arrived)
            event = torch.cuda.Event()
            event.record()
            self.free_again[turn] = event
        return out

    def close(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            self.pool.shutdown()
            self.buffers = []


def load_checkpoint(model, model_dir: str) -> None:
    """Reads ``model_dir`` and hands the model its tensors on ``model.env.device``."""
    files = ModelFiles(model_dir)
    manifest = model.manifest()
    check_against_manifest({name: (e.dtype, e.shape) for name, e in files.entries.items()}, manifest)
    env = model.env
    tensors: Dict[str, torch.Tensor] = {}
    uploader = Uploader(env.device)
    try:
        for name, (param, _) in manifest.items():
            if name not in files.entries:
                continue
            tensors[name] = uploader.upload(files.read(name), device_dtype(param, env.dtype))
    finally:
        uploader.close()
    model.load(tensors)


def load_tensors(model, named_tensors) -> None:
    """Same as :func:`load_checkpoint` for tensors that already exist (random initialisation)."""
    manifest = model.manifest()
    env = model.env
    tensors: Dict[str, torch.Tensor] = {}
    seen: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
    for name, value in named_tensors:
        seen[name] = (value.dtype, tuple(value.shape))
        if name in manifest and tuple(value.shape) == tuple(manifest[name][0].shape):
            tensors[name] = value.to(device=env.device, dtype=device_dtype(manifest[name][0], env.dtype)).contiguous()
    check_against_manifest(seen, manifest)
    model.load(tensors)


def write_model_folder(out_dir: str, raw_config: dict, named_tensors) -> None:
    """Writes ``config.json`` and ``model.safetensors``."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(raw_config, handle, indent=2)
        handle.write("\n")
    write_safetensors(os.path.join(out_dir, "model.safetensors"), {n: t.cpu() for n, t in named_tensors},
                      metadata={"format": "pt"})

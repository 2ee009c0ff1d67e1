"""Reading and writing safetensors files by tensor name.

The file format is: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets"}}``, then the raw little-endian
tensor bytes.  The reader maps the file and hands out zero-copy views, in the
manner of the reference's mmap-backed ``gguf::File`` (src/models/gguf.cpp:411,
:563); a folder may hold one ``model.safetensors`` or shards listed in
``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightFileError(RuntimeError):
    """A safetensors file that cannot be parsed."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int          # byte offset in the file
    end: int
    path: str


class SafetensorsFile:
    """One mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightFileError(f"{path}: too short to be a safetensors file")
        self._handle = open(path, "rb")
        # A private copy-on-write mapping: torch wants a writable buffer, and
        # nothing is ever written through it.
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_COPY)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len <= 0 or 8 + header_len > size:
            raise WeightFileError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise WeightFileError(f"{path}: header is not JSON ({error})") from error
        base = 8 + header_len
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(d) for d in info["shape"])
                begin, end = (int(o) for o in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as error:
                raise WeightFileError(f"{path}: bad header entry for '{name}' ({error})") from error
            count = 1
            for d in shape:
                count *= d
            if end - begin != count * dtype.itemsize or begin < 0 or base + end > size:
                raise WeightFileError(
                    f"{path}: tensor '{name}' claims bytes [{begin},{end}) for shape {list(shape)} "
                    f"{info['dtype']}, which does not fit the file")
            self.entries[name] = TensorEntry(name, dtype, shape, base + begin, base + end, path)

    def read(self, name: str) -> torch.Tensor:
        entry = self.entries[name]
        count = 1
        for d in entry.shape:
            count *= d
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        flat = torch.frombuffer(self._map, dtype=entry.dtype, count=count, offset=entry.begin)
        return flat.view(entry.shape)


class ModelFiles:
    """All tensors of a model folder, by name, whichever shard holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        paths: List[str] = []
        if os.path.isfile(index_path):
            with open(index_path, "r", encoding="utf-8") as handle:
                index = json.load(handle)
            shard_names = sorted(set(index.get("weight_map", {}).values()))
            if not shard_names:
                raise WeightFileError(f"{index_path}: empty weight_map")
            paths = [os.path.join(model_dir, s) for s in shard_names]
        elif os.path.isfile(single):
            paths = [single]
        else:
            raise WeightFileError(f"{model_dir}: no model.safetensors (nor model.safetensors.index.json)")
        self.files = [SafetensorsFile(p) for p in paths]
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        for shard in self.files:
            for name, entry in shard.entries.items():
                if name in self.entries:
                    raise WeightFileError(f"tensor '{name}' appears in both {self.entries[name].path} and {shard.path}")
                self.entries[name] = entry
                self._owner[name] = shard

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Writes ``tensors`` (CPU, any supported dtype) in name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered = sorted(tensors.items())
    for name, tensor in ordered:
        if tensor.dtype not in _NAMES:
            raise WeightFileError(f"tensor '{name}': dtype {tensor.dtype} cannot be stored")
        nbytes = tensor.numel() * tensor.dtype.itemsize
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - (len(blob) + 8) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name, tensor in ordered:
            data = tensor.detach().contiguous().cpu()
            if data.numel():
                handle.write(memoryview(data.reshape(-1).view(torch.uint8).numpy()))

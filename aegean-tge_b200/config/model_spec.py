"""Architecture-independent description of a decoder.

An architecture module (for instance ``models/qwen2.py``) turns its typed
configuration into a :class:`ModelSpec`.  The generic decoder in
``models/decoder.py`` builds itself from the spec alone: it never looks at an
architecture name.  Everything a part needs (sizes, eps, rope base, bias
flags) travels in ``PartSpec.params``; the checkpoint tensor names a part
binds travel in ``PartSpec.weights`` (local parameter name -> tensor name in
the safetensors file), so parts know neither the model nor the file layout.

The reference hard-codes one layer body three times
(src/models/qwen2.cpp:2032-2123, :2130-2500, :1613-1946); here the same body
is data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: which registered kind, with which parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    weights: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement ("block") of a mixer and a feed-forward.

    ``cache_from`` names another layer (by its index in ``ModelSpec.layers``)
    whose cache this layer's mixer reads instead of writing one of its own.
    """

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """The whole decoder as data.

    ``schedule`` is the order in which layers run, as indices into ``layers``;
    a layer may be named twice (its weights and cache are then shared between
    the two visits only if the mixer allows it) and the list need not be
    ``range(len(layers))``.
    """

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[int, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    end_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if self.hidden_size <= 0 or self.vocab_size <= 0 or self.max_positions <= 0:
            raise ValueError("model spec: hidden_size, vocab_size and max_positions must be positive")
        if not self.layers:
            raise ValueError("model spec: no layers")
        for step, index in enumerate(self.schedule):
            if not 0 <= index < len(self.layers):
                raise ValueError(f"model spec: schedule[{step}]={index} names no layer")
        for index, layer in enumerate(self.layers):
            if layer.cache_from is not None:
                if not 0 <= layer.cache_from < len(self.layers) or layer.cache_from == index:
                    raise ValueError(f"model spec: layer {index} reads the cache of layer "
                                     f"{layer.cache_from}, which does not exist")
                if self.layers[layer.cache_from].cache_from is not None:
                    raise ValueError(f"model spec: layer {index} reads the cache of layer "
                                     f"{layer.cache_from}, which has no cache of its own")
                first_self = self.schedule.index(index) if index in self.schedule else None
                first_src = (self.schedule.index(layer.cache_from)
                             if layer.cache_from in self.schedule else None)
                if first_self is not None and (first_src is None or first_src > first_self):
                    raise ValueError(f"model spec: layer {index} runs before layer "
                                     f"{layer.cache_from} has written the cache it reads")


def expected_tensors(spec: ModelSpec) -> Dict[str, str]:
    """Checkpoint tensor name -> "where it is used", for error messages."""
    names: Dict[str, str] = {}
    def add(part: PartSpec, where: str) -> None:
        for local, name in part.weights.items():
            names.setdefault(name, f"{where}.{local}")
    add(spec.embedding, "embedding")
    add(spec.final_norm, "final_norm")
    add(spec.head, "head")
    for index, layer in enumerate(spec.layers):
        add(layer.mixer_norm, f"layers[{index}].mixer_norm")
        add(layer.mixer, f"layers[{index}].mixer")
        add(layer.ffn_norm, f"layers[{index}].ffn_norm")
        add(layer.feed_forward, f"layers[{index}].feed_forward")
    return names

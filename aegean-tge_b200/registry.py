"""One registry from an architecture's name to its model.

``config.json`` names the architecture in ``architectures[0]``; the entry
registered under that name turns the raw config into a typed configuration
and the typed configuration into a :class:`ModelSpec`.  The reference has no
registry: one class serves every file and the architecture string only flips
two switches (src/models/qwen2.cpp:253-258, :331-336).  Here the name picks
everything, and an unknown name is an error that lists the known ones.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Tuple

from .config.model_spec import ModelSpec
from .config.common import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]
    # typed config -> (tensor name, shape, role "matrix" | "vector", weights.draws.Draw) of every checkpoint
    # tensor: what the random-weights mode draws (weights/random_init.py)
    random_plan: Callable[[Any], Iterable[Tuple[str, Tuple[int, ...], str, Any]]]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(entry: Architecture) -> None:
    if entry.name in _ARCHITECTURES:
        raise ValueError(f"architecture '{entry.name}' is already registered")
    _ARCHITECTURES[entry.name] = entry


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(raw_config: Dict[str, Any]) -> Architecture:
    names = raw_config.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: missing key 'architectures' (a list with the model class name)")
    name = names[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture '{name}' is not registered; "
                          f"registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]

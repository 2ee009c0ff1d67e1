"""What every architecture's configuration shares: the error type and the reading of config.json."""
from __future__ import annotations

import json
import os
from typing import Any, Dict


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
    except json.JSONDecodeError as error:
        raise ConfigError(f"{path}: not valid JSON ({error})") from error
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw

"""Typed configurations and the architecture-independent model description."""
from .model_spec import LayerSpec, ModelSpec, PartSpec, expected_tensors
from .qwen2 import ARCHITECTURE as QWEN2_ARCHITECTURE
from .common import ConfigError, read_config_json
from .qwen2 import Qwen2Config

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "expected_tensors", "ConfigError",
           "Qwen2Config", "QWEN2_ARCHITECTURE", "read_config_json"]

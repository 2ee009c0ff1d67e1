"""Model assembly.  Importing this package registers the architectures it holds."""
from . import qwen2  # noqa: F401  (registration)
from .decoder import DecoderModel

__all__ = ["DecoderModel"]

"""A small, whole inference engine for one B200: Qwen2.5 dense decoder, from token ids to next token.

Public entry points:

* :class:`Engine` - load a model folder (or random weights) and generate;
* :class:`SamplingParams` - sampling controls;
* :func:`write_random_model` - a model folder from a configuration and a seed;
* ``bin/tge`` and ``bin/trace_run`` - the command line and trace replay.
"""
from . import models as _models  # noqa: F401  (registers architectures)
from . import parts as _parts    # noqa: F401  (registers parts)
from .config import ConfigError, Qwen2Config
from .registry import architecture_of, register_architecture, registered_architectures
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__version__ = "0.1.0"


def __getattr__(name):
    # The engine pulls in the CUDA bindings; keep `import aegean_tge_b200` light for host-only use.
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)


__all__ = ["Engine", "SamplingParams", "ConfigError", "Qwen2Config", "WeightError", "write_random_model",
           "architecture_of", "register_architecture", "registered_architectures", "__version__"]

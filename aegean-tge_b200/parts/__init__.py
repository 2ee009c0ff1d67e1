"""Parts a layer is put together from.  Importing this package registers the built-in ones."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, FeedForward,
                   LayerCache, Mixer, Norm, PagedCacheSpec, ParamSpec, Part, PositionEncoding, StateSpec, StepContext,
                   build_part)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv",
           "FeedForward", "LayerCache", "Mixer", "Norm", "PagedCacheSpec", "ParamSpec", "Part", "PositionEncoding",
           "StateSpec", "StepContext", "build_part"]

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext,
                   CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, Registry, StateNeed)
from . import attention, block, embedding, rmsnorm, rope, swiglu  # noqa: F401  (register the built-in parts)
from .block import Block

__all__ = ["Block", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
           "BuildContext", "CacheNeed", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding",
           "Registry", "StateNeed"]

"""Parts a decoder is put together from.  Importing this package registers the built-in kinds."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVNeed,
                   LayerSpec, Mixer, ModelSpec, Norm, ParamSpec, Part, PartSpec, PositionEncoding, Registry,
                   RunSpec, StateNeed)
from . import attention, block, mlp, norm, rotary  # noqa: F401  (registration)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "FeedForward",
           "KVNeed", "LayerSpec", "Mixer", "ModelSpec", "Norm", "ParamSpec", "Part", "PartSpec",
           "PositionEncoding", "Registry", "RunSpec", "StateNeed"]

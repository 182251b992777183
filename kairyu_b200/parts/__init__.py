"""Model parts and their registries.  Importing this package registers the
built-in parts; more can be registered from outside with the same decorators."""

from kairyu_b200.parts import attention, block, embedding, ffn, norm, rope  # noqa: F401  (registration)
from kairyu_b200.parts.base import (
    BLOCKS,
    EMBEDDINGS,
    FEED_FORWARDS,
    HEADS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Block,
    CacheView,
    FeedForward,
    LayerCall,
    LayerSpec,
    Mixer,
    ModelSpec,
    Norm,
    PagedKVSpec,
    Part,
    PartSpec,
    PositionEncoding,
    StateSpec,
    StepContext,
    TensorSpec,
)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "CacheView", "FeedForward", "LayerCall", "LayerSpec", "Mixer", "ModelSpec", "Norm",
    "PagedKVSpec", "Part", "PartSpec", "PositionEncoding", "StateSpec", "StepContext", "TensorSpec",
]

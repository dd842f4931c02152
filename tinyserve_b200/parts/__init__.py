"""The parts layers are assembled from. Importing the package registers the built-in ones."""

from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    Block, CacheNeed, FeedForward, KVCacheEntry, KVGroupContext, KVNeed, Mixer, Norm, PagedNeed, Part,
    PositionEncoding, ResidualStream, Rotation, SlotNeed, StateCacheEntry, StateNeed, StepContext, TensorSpec,
    register_block, register_feed_forward, register_mixer, register_norm,
    register_position_encoding,
)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
    "Block", "CacheNeed", "FeedForward", "KVCacheEntry", "KVGroupContext", "KVNeed", "Mixer", "Norm", "PagedNeed",
    "Part", "PositionEncoding", "ResidualStream", "Rotation", "SlotNeed", "StateCacheEntry", "StateNeed", "StepContext",
    "TensorSpec", "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position_encoding",
]

"""The parts that layers are put together from, and their registries."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                   CacheNeed, Part, StateNeed, TensorNeed, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (register)
from .linear import Linear

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS",
           "CacheNeed", "Part", "StateNeed", "TensorNeed", "Linear", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position"]

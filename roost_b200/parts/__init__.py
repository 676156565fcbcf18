"""Parts a model is assembled from. Importing the package registers the built-in kinds."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CacheNeed, FeedForward, Mixer, Norm, ParamDecl,
                   Part, Runtime, register_block, register_feed_forward, register_mixer, register_norm, register_position)
from . import attention, block, mlp, norms, positions  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheNeed", "FeedForward", "Mixer", "Norm",
           "ParamDecl", "Part", "Runtime", "Linear", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position"]

"""Parts a model is assembled from. Importing the package registers the built-in kinds."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, CacheNeed, Embedding, FeedForward, Head,
                   Mixer, Norm, ParamDecl, Part, Runtime, register_block, register_embedding, register_feed_forward, register_head,
                   register_mixer, register_norm, register_position)
from . import attention, block, mlp, norms, positions, vocab  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheNeed", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "ParamDecl", "Part", "Runtime", "Linear", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position"]

"""Parts a model is put together from; importing this package registers the built-in ones."""
from . import attention, block, embedding, feed_forward, head, norm, rotary  # noqa: F401
from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                       POSITION_ENCODINGS, BuildContext, WeightAccess, lookup, register_block,
                       register_embedding, register_feed_forward, register_head, register_mixer,
                       register_norm, register_position_encoding)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
           "BuildContext", "WeightAccess", "lookup", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position_encoding"]

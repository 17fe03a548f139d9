from . import attention, block, embedding, feedforward, norm, position  # noqa: F401 (register)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                   ResidualStream, Runtime, make_part, register_block, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from .model import Model

__all__ = ["Model", "Runtime", "ResidualStream", "MIXERS", "FEED_FORWARDS", "NORMS",
           "POSITIONS", "BLOCKS", "EMBEDDINGS", "HEADS", "make_part", "register_mixer",
           "register_feed_forward", "register_norm", "register_position", "register_block",
           "register_embedding", "register_head"]

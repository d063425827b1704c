from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Runtime, register_block,
                   register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from . import attention, block, delta, embedding, feed_forward, latent_attention, linear_attention, moe, norm, parallel, position, ssm, time_mix  # noqa: F401  (registers the kinds)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Runtime", "register_block",
           "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position"]

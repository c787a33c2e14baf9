from .registry import (BLOCKS, EMBEDDING_ADDENDS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup, register_block,
                       register_embedding_addend, register_feed_forward, register_mixer, register_norm, register_position)
from .runtime import Runtime, Workspace
from . import (attention, block, delta_rule, embedding, feed_forward, hyper, latent_attention, linear_attention,  # registers
               moe, norm, parallel, position, recurrence, rotary_attention, sink_attention)                         # the built-in parts

__all__ = ["BLOCKS", "EMBEDDING_ADDENDS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "lookup", "register_block",
           "register_embedding_addend", "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "Runtime", "Workspace"]

from .base import (CacheNeed, Embedder, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   embedder_class, feed_forward_class, mixer_class, norm_class, position_class,
                   register_embedder, register_feed_forward, register_mixer, register_norm, register_position)
from . import (attention, embedding, latent_attention, mlp, norm, rotary,  # noqa: F401  (register the built-in kinds)
               state_space)
from .block import Block, arrangement, register_arrangement

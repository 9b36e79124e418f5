from .base import (CacheNeed, Embedder, FeedForward, Mixer, Norm, NormedDelta, Part, PositionEncoding, StateNeed,
                   embedder_class, feed_forward_class, mixer_class, norm_class, position_class,
                   register_embedder, register_feed_forward, register_mixer, register_norm, register_position)
from . import (attention, delta_rule, diff_attention, embedding, latent_attention, mlp, norm,  # noqa: F401  (register
               rotary, state_space)                                                            # the built-in kinds)
from .block import Block, arrangement, register_arrangement

from .base import (CacheNeed, Embedder, FeedForward, Mixer, Norm, NormedDelta, Part, PositionEncoding, StateNeed, SummedDelta,
                   embedder_class, feed_forward_class, mixer_class, norm_class, position_class,
                   register_embedder, register_feed_forward, register_mixer, register_norm, register_position)
from . import (attention, delta_rule, diff_attention, embedding, latent_attention, mixer_pair, mlp, moe, norm,  # noqa: F401  (register
               rotary, state_space, talking_attention, time_mix)                                                            # the built-in kinds)
from .block import Block, SublayerGate, arrangement, register_arrangement

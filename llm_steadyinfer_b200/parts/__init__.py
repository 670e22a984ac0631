from .base import (CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   feed_forward_class, mixer_class, norm_class, position_class,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import attention, mlp, norm, rotary  # noqa: F401  (register the built-in kinds)
from .block import Block, arrangement, register_arrangement

from . import attention, block, mlp, norm, rope  # noqa: F401  (registers the kinds)
from .base import Block, CacheNeed, FeedForward, Mixer, Norm, Part
from .linear import StackedLinear
from .model import DecoderModel
from .registry import (build, register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, unregister)

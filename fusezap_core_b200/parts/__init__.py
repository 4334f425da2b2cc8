from .base import (MIXERS, FEED_FORWARDS, NORMS, POSITIONS, BLOCKS, LOGIT_TRANSFORMS, register_mixer, register_feed_forward,
                   register_norm, register_position, register_block, register_logit_transform, build, LayerCache, Part,
                   Mixer, FeedForward, Norm, PositionEncoding, Block, LogitTransform)
from . import rope, norm, attention, feed_forward, block   # registers the dense decoder's parts

__all__ = ["MIXERS", "FEED_FORWARDS", "NORMS", "POSITIONS", "BLOCKS", "LOGIT_TRANSFORMS", "register_mixer",
           "register_feed_forward", "register_norm", "register_position", "register_block", "register_logit_transform",
           "build", "LayerCache", "Part", "Mixer", "FeedForward", "Norm", "PositionEncoding", "Block", "LogitTransform"]

"""Parts a model is put together from, and the model assembled from them."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheView,
                   FeedForward, GroupContext, KVPagesNeed, Mixer, Norm, Part, PartEnv,
                   PositionEncoding, StateNeed, StepContext, WeightInfo)
from .model import DecoderModel
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheView",
    "DecoderModel", "FeedForward", "GroupContext", "KVPagesNeed", "LayerSpec", "Mixer", "ModelSpec",
    "Norm", "Part", "PartEnv", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateNeed",
    "StepContext", "WeightInfo",
]

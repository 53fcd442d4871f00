"""Parts a model is put together from, and the model assembled from them."""

from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS, OUTPUT_HEADS, POSITION_ENCODINGS, Block,
                   CacheView, Embedding, FeedForward, GroupContext, KVPagesNeed, Mixer, Norm, OutputHead, Part,
                   PartEnv, PositionEncoding, StateNeed, StepContext, WeightInfo)
from .model import DecoderModel
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "MIXERS", "NORMS", "OUTPUT_HEADS", "POSITION_ENCODINGS", "Block",
    "CacheView", "DecoderModel", "Embedding", "FeedForward", "GroupContext", "KVPagesNeed", "LayerSpec", "Mixer", "ModelSpec",
    "Norm", "OutputHead", "Part", "PartEnv", "PartSpec", "PositionEncoding", "ScheduleEntry", "StateNeed",
    "StepContext", "WeightInfo",
]

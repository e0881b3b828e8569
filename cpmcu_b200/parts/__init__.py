"""Parts a model is assembled from.  Importing this package registers the built-in ones."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CacheNeeds, FeedForward, LayerSpec,
                   Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, Registry, ResidualStream,
                   ScheduleEntry, StepContext, WeightSpec, build_block, build_part, default_schedule)
from .embedding import EMBEDDINGS, HEADS
from . import attention, block, feedforward, norm, position  # noqa: F401  (registration)

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "EMBEDDINGS", "HEADS", "Block", "CacheNeeds",
    "FeedForward", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec", "PositionEncoding", "Registry",
    "ResidualStream", "ScheduleEntry", "StepContext", "WeightSpec", "build_block", "build_part",
    "default_schedule",
]

"""Layer parts and the model assembled from them."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (register the built-in parts)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FoldedInput, NormFold, PagedKVNeed, ResidualAdd, ParamSpec, Part, StateNeed,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position)
from .context import PagedKVView, StateView, StepContext
from .model import CacheGroup, DecoderModel, RunCache
from .spec import LayerRun, LayerSpec, ModelSpec, PartSpec

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "FoldedInput", "NormFold", "PagedKVNeed", "ResidualAdd", "ParamSpec", "Part",
           "StateNeed", "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "PagedKVView", "StateView", "StepContext", "CacheGroup", "DecoderModel", "RunCache",
           "LayerRun", "LayerSpec", "ModelSpec", "PartSpec"]

from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext, Workspace
from .registry import build_block, build_part, register_part, registered_parts
from . import attention, block, embedding, feed_forward, norm, position  # registers the built-in parts
from .model import DecoderModel

__all__ = [
    "CacheNeed", "DecoderModel", "LaneView", "Part", "StateNeed", "StepContext", "WeightSpec", "Workspace",
    "build_block", "build_part", "register_part", "registered_parts",
]

from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the parts)
from .base import (CacheNeed, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, Runtime, StateNeed, StepContext)
from .registry import make_part, register_part, registered_parts
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = ["CacheNeed", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "StateNeed",
           "StepContext", "make_part", "register_part", "registered_parts", "LayerSpec", "ModelSpec",
           "PartSpec", "ScheduleEntry"]

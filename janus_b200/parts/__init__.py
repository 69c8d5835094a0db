from . import attention, block, feedforward, norm, rope  # noqa: F401  (registers the built-in kinds)
from .base import (FeedForward, KVSpec, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, StateSpec, make_part, register_part,
                   registered_parts)

__all__ = [
    "FeedForward", "KVSpec", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec",
    "PositionEncoding", "ScheduleEntry", "StateSpec", "make_part", "register_part", "registered_parts",
]

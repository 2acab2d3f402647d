from .base import (FeedForward, LayerCache, Mixer, Norm, Part, PositionEncoding, StepContext,
                   Workspace, build_part, register_part, registered_parts)
from . import attention, embedding, feed_forward, norm, position  # noqa: F401  (register kinds)

__all__ = [
    "FeedForward", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext",
    "Workspace", "build_part", "register_part", "registered_parts",
]

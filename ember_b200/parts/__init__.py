"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, arrangements."""
from .base import CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, WeightDecl
from .registry import build_part, part_class, register_part, registered_parts
from .linear import Linear
from . import norm, position, attention, feedforward, block  # noqa: F401  (registers the built-in parts)

__all__ = ["CacheNeed", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "WeightDecl",
           "build_part", "part_class", "register_part", "registered_parts", "Linear"]

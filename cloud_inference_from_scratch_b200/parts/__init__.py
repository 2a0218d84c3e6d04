from . import attention, block, mlp, norm, rotary  # noqa: F401  (registers the built-in parts)
from .base import (
    Block,
    CacheSpec,
    FeedForward,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    StateSpec,
    TensorSpec,
    build_part,
    part_class,
    register_part,
    registered_parts,
)

__all__ = [
    "Block", "CacheSpec", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateSpec", "TensorSpec", "build_part", "part_class", "register_part", "registered_parts",
]

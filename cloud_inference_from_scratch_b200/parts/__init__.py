from . import attention, block, connection, delta, latent, lightning, mlp, norm, rotary, routed  # noqa: F401  (registers the built-in parts)
from .base import (
    Block,
    CacheSpec,
    Connection,
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
    "Block", "CacheSpec", "Connection", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "StateSpec", "TensorSpec", "build_part", "part_class", "register_part", "registered_parts",
]

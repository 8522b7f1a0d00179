"""Parts a model is assembled from. Importing this package registers the built-in kinds."""

from matricxon_b200.parts import attention, block, mlp, norm, rotary  # noqa: F401  (registration)
from matricxon_b200.parts.base import (
    Block,
    CacheBinding,
    FeedForward,
    KVCacheRequest,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    Runtime,
    StateRequest,
    build_part,
    part_class,
    register_part,
)

__all__ = ["Block", "CacheBinding", "FeedForward", "KVCacheRequest", "Mixer", "Norm", "Part",
           "PositionEncoding", "Runtime", "StateRequest", "build_part", "part_class",
           "register_part"]

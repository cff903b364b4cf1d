"""Importing this package registers the parts the framework ships."""
from . import attention, embedding, mlp, norm, rope  # noqa: F401
from .base import (CacheView, FeedForward, GroupTables, HalfRotation, Mixer, Norm, PagedKVNeed, Part, PositionEncoding, StateNeed,
                   StepContext)

__all__ = ["CacheView", "FeedForward", "GroupTables", "HalfRotation", "Mixer", "Norm", "PagedKVNeed", "Part", "PositionEncoding",
           "StateNeed", "StepContext"]

"""Architectures: each module registers its builder (config.json -> ModelSpec) by name."""

from . import dense_swiglu  # noqa: F401
from .decoder import CacheEntryPlan, DecoderModel

__all__ = ["CacheEntryPlan", "DecoderModel"]

from .decoder import DecoderConfig, RopeScaling
from .generation import GenerationConfig, GenerationOverrides, GenerationSettings, DEFAULT_SEED
from .runtime import CacheConfig, CudaConfig, RuntimeConfig, SchedulerConfig
from .spec import (CacheRequirement, EmbeddingSpec, FixedState, HeadSpec, LayerSpec, ModelSpec, PagedKv,
                   ParamSpec, ScheduleEntry)

__all__ = [
    "DecoderConfig", "RopeScaling", "GenerationConfig", "GenerationOverrides", "GenerationSettings",
    "DEFAULT_SEED", "CacheConfig", "CudaConfig", "RuntimeConfig", "SchedulerConfig", "CacheRequirement",
    "EmbeddingSpec", "FixedState", "HeadSpec", "LayerSpec", "ModelSpec", "PagedKv", "ParamSpec", "ScheduleEntry",
]

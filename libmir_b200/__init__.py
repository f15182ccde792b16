"""libmir_b200: a single-GPU inference engine for the dense SwiGLU decoder on NVIDIA B200 (sm_100a).

    from libmir_b200 import Library, RuntimeConfig, GenerationRequest, GenerationOverrides
    model = Library(RuntimeConfig()).load("/path/to/model")
    out = model.generate(GenerationRequest(prompt_ids=[1, 2, 3], options=GenerationOverrides(max_tokens=16)))
"""

from .config import (CacheConfig, CudaConfig, DecoderConfig, GenerationConfig, GenerationOverrides,
                     GenerationSettings, RuntimeConfig, SchedulerConfig)
from .engine import (GenerationOutput, GenerationRequest, Library, Model, SamplingLogits, Session, StepEntry,
                     StepResult)
from .errors import (ConfigError, KernelError, KvCachePressure, KvCapacity, LibmirError, NoFreeSlot, RegistryError,
                     SchedulerError, WeightsError)
from .registry import build_spec, known_architectures, register_architecture, register_part

__version__ = "0.1.0"

__all__ = [
    "CacheConfig", "ConfigError", "CudaConfig", "DecoderConfig", "GenerationConfig", "GenerationOutput",
    "GenerationOverrides", "GenerationRequest", "GenerationSettings", "KernelError", "KvCachePressure", "KvCapacity",
    "LibmirError", "Library", "Model", "NoFreeSlot", "RegistryError", "RuntimeConfig", "SamplingLogits",
    "SchedulerConfig", "SchedulerError", "Session", "StepEntry", "StepResult", "WeightsError", "build_spec",
    "known_architectures", "register_architecture", "register_part",
]

from .rng import SplitMix64
from .sampler import DeviceSampler, RequestSampler

__all__ = ["DeviceSampler", "RequestSampler", "SplitMix64"]

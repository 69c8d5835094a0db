from .params import SamplerConfig
from .sampler import DeviceSampler

__all__ = ["SamplerConfig", "DeviceSampler"]

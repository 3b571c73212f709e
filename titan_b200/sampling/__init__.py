from .params import DEFAULT_SEED, GREEDY_TEMPERATURE, SamplerParams
from .sampler import DeviceSampler

__all__ = ["DEFAULT_SEED", "GREEDY_TEMPERATURE", "SamplerParams", "DeviceSampler"]

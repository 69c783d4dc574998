from .params import SamplingParams
from .rng import Xoshiro256StarStar
from .sampler import DeviceSampler, RequestSampler

__all__ = ["SamplingParams", "Xoshiro256StarStar", "DeviceSampler", "RequestSampler"]

from .params import InvalidSamplingParams, SamplingParams
from .sampler import Sampler, SamplingRow

__all__ = ["InvalidSamplingParams", "SamplingParams", "Sampler", "SamplingRow"]

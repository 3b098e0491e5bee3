from .params import SamplingParams
from .sampler import Sampler, uniform_for

__all__ = ["SamplingParams", "Sampler", "uniform_for"]

from .params import SamplingParams
from .sampler import Sampler, PendingTokens, uniform_for

__all__ = ["SamplingParams", "Sampler", "PendingTokens", "uniform_for"]

"""Sampling: parameters, the device selector, and its host restatement."""
from .params import SamplingParams
from .sampler import Sampler, gumbel_scores, stream_key, uniform24

__all__ = ["SamplingParams", "Sampler", "gumbel_scores", "stream_key", "uniform24"]

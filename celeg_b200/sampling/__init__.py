"""Greedy, temperature, top-k, top-p and repetition-penalty sampling."""
from .params import GREEDY, MAX_TOP_K, SamplingParams
from .sampler import Sampler

__all__ = ["GREEDY", "MAX_TOP_K", "SamplingParams", "Sampler"]

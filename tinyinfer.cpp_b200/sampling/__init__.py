"""Greedy and temperature / top-k / top-p sampling."""
from .params import SamplingParams
from .sampler import Sampler, uniform

__all__ = ["Sampler", "SamplingParams", "uniform"]

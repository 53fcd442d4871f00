"""Sampling options and the sampler."""

from .params import GREEDY_EPS, SamplingParams
from .sampler import Sampler

__all__ = ["GREEDY_EPS", "SamplingParams", "Sampler"]

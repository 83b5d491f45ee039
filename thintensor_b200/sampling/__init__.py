"""Greedy, temperature, top-k and top-p sampling."""
from .sampler import SamplingParams, sample

__all__ = ["SamplingParams", "sample"]

"""Greedy, temperature and top-p sampling."""
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]

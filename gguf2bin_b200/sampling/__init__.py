"""Sampling: greedy, temperature, and the reference's top-k / top-p / repeat penalty."""
from .params import RECENT_USE, SamplingParams
from .sampler import Sampler

__all__ = ["RECENT_USE", "SamplingParams", "Sampler"]

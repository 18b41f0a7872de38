"""Sampling: greedy, temperature, top-k and top-p, on the device."""
from .sampler import Sampler, SamplingParams, uniform01

__all__ = ["Sampler", "SamplingParams", "uniform01"]

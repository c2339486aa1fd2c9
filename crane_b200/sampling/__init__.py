"""Sampling: greedy, temperature, top-k, top-p, repetition penalty."""
from .sampler import Sampler, SamplingParams

__all__ = ["Sampler", "SamplingParams"]

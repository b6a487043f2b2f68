"""Sampling: greedy, temperature, nucleus and repeat penalty, on the device."""
from .sampler import Sampler, SamplingParams, seed_state

__all__ = ["Sampler", "SamplingParams", "seed_state"]

"""Sampling: options in the reference's names, and the device sampler."""
from .params import SamplingParams
from .sampler import Sampler

__all__ = ["SamplingParams", "Sampler"]

"""Sampling parameters, the per-request random stream, and the device sampler."""
from .params import DEFAULT_SEED, SamplingParams, XorShift32
from .sampler import Sampler

__all__ = ["DEFAULT_SEED", "SamplingParams", "XorShift32", "Sampler"]

"""Sampling: parameters and the device sampler."""
from .params import SamplingParams
from .sampler import Sampler, SamplerState, splitmix64, uniform01

__all__ = ["SamplingParams", "Sampler", "SamplerState", "splitmix64", "uniform01"]

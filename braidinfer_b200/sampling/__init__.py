"""Sampling: options, counter-based uniform numbers, the device sampler."""
from .params import SamplingParams
from .rng import entropy_seed, uniform
from .sampler import Sampler

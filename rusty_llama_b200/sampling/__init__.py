"""Sampling: greedy, temperature, top-p, seeded."""

from .sampler import Sampler, SamplingParams, default_seed, sequence_seed

__all__ = ["Sampler", "SamplingParams", "default_seed", "sequence_seed"]

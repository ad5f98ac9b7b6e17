"""Sampling options and the device sampler."""

from turingserve_b200.sampling.params import SamplingParams
from turingserve_b200.sampling.sampler import Sampler, SampleRow, derive_seed

__all__ = ["SamplingParams", "Sampler", "SampleRow", "derive_seed"]

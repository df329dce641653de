"""Sampling: options, the host statement of the semantics, and the device kernel."""
from .params import SamplingParams
from .host import gumbel_noise, sample_host, sampling_distribution

__all__ = ["SamplingParams", "gumbel_noise", "sample_host", "sampling_distribution"]

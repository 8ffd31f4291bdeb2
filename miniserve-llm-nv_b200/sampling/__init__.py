"""Sampling parameters; the sampler itself is a device kernel (``kernels.sample``)."""

from .params import SamplingParams

__all__ = ["SamplingParams"]

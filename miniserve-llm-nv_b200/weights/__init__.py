"""Weights: strict loading by tensor name, and seeded random model folders."""

from .loader import WeightLoadError, WeightLoadReport, load_tensors
from .random_init import random_tensors, write_random_model

__all__ = ["WeightLoadError", "WeightLoadReport", "load_tensors", "random_tensors", "write_random_model"]

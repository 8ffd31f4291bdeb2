"""Norm parts.  ``rms``: ``weight * x * rsqrt(mean(x^2) + eps)`` with the statistics in float32
(miniserve/model/layers.py:30-34), fused with the residual add that precedes it."""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_norm


@register_norm("rms")
class RMSNorm(Part):
    def __init__(self, *, name: str, size: int, eps: float, prefix: str = "") -> None:
        self.name, self.size, self.eps = prefix + name, size, float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "vector")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def add_and_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                     rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += delta`` (float32, in place; skipped when ``delta`` is None), ``out = norm(residual)``.

        With ``rows`` only those rows are normalised into ``out [len(rows), size]`` and the
        residual stays as it is.
        """
        kernels.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out

    def fold(self) -> tuple[torch.Tensor, float]:
        """(weight, eps): all that the products around this norm need to carry it out between them."""
        return self.weight, self.eps

    def norm(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Norm over the last dim of ``x`` (any leading shape) without a residual."""
        kernels.rmsnorm(x, self.weight, self.eps, out)
        return out

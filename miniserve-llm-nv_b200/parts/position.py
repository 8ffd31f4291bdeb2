"""Position encodings applied to queries and keys inside the attention mixer.

``rope``: rotation by ``position * theta^(-2j/rotary_dim)`` (miniserve/model/rope.py:24-52),
half-split pairing ``(j, j + rotary_dim/2)`` by default, interleaved pairing ``(2j, 2j+1)`` or
a rotary size below the head size as options.  Angles, cosines and sines are float32 and are
computed once per step for all layers that share the same encoding.
``none``: no position encoding.

A position part either offers ``fused_args(ctx)``, the arguments of the fused
norm+rotation+append kernel, or returns None there and implements ``apply(q, k, ctx)``, which the
mixer calls on the projected heads before they are appended.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Part, register_position
from .context import StepContext


@register_position("rope")
class RotaryPosition(Part):
    def __init__(self, *, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 interleaved: bool = False) -> None:
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        self.interleaved = bool(interleaved)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and within the head size {head_dim}")
        self._inv_freq: Optional[torch.Tensor] = None

    def inv_freq(self, device) -> torch.Tensor:
        """``1 / theta ** (arange(0, rotary_dim, 2) / rotary_dim)`` in float32 (rope.py:24-25)."""
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            self._inv_freq = (1.0 / (self.theta ** exponents)).to(device)
        return self._inv_freq

    def tables(self, ctx: StepContext) -> torch.Tensor:
        """float32 ``[N, rotary_dim/2, 2]`` of (cos, sin), shared through the step's memo."""
        key = ("rope", self.theta, self.rotary_dim)
        table = ctx.memo.get(key)
        if table is None:
            table = torch.empty((ctx.n_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=ctx.device)
            kernels.rope_table(ctx.positions, self.inv_freq(ctx.device), table)
            ctx.memo[key] = table
        return table

    def fused_args(self, ctx: StepContext):
        return self.tables(ctx), self.rotary_dim, self.interleaved


@register_position("none")
class NoPosition(Part):
    def __init__(self, **_ignored) -> None:
        pass

    def fused_args(self, ctx: StepContext):
        return None, 0, False

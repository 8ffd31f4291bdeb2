"""Block arrangements.  ``pre_norm``: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
(miniserve/model/qwen3.py:336-346).

The residual stream ``h`` is float32 and is updated in place.  A block receives the stream
together with a *pending* ``delta`` that has not been added yet (the previous block's
feed-forward output) and returns its own pending delta, so that every residual add is fused
into the norm that follows it.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from .base import register_block
from .context import StepContext


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx: StepContext, cache: Any) -> torch.Tensor:
        normed = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
        self.mixer_norm.add_and_norm(residual, delta, normed)
        delta = self.mixer.forward(normed, ctx, cache)
        normed = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
        self.feed_forward_norm.add_and_norm(residual, delta, normed)
        return self.feed_forward.forward(normed, ctx)

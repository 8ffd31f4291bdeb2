"""Block arrangements.  ``pre_norm``: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
(miniserve/model/qwen3.py:336-346).

The residual stream ``h`` is float32 and is updated in place.  A block receives the stream
together with a *pending* ``delta`` that has not been added yet (the previous block's
feed-forward output) and returns its own pending delta, so that every residual add is fused
into the norm that follows it.

In steps of few rows (decode steps) a norm and the add before it cost two kernels that do next
to nothing.  Where the parts on both sides offer it (``parts.base``: ``fold_output_weight``,
``fold``, ``fold_input_weight``) the block leaves them out: the product before the norm adds
into the stream itself and writes ``h * norm weight`` with the rows' sums of squares, and the
product behind the norm divides its own results by the rows' root mean square.  What is handed
on is then a :class:`~.base.FoldedInput` instead of a delta.
"""

from __future__ import annotations

from typing import Any, Optional, Union

import torch

from .. import kernels
from .base import FoldedInput, NormFold, ResidualAdd, register_block
from .context import StepContext

Pending = Union[None, torch.Tensor, FoldedInput]     # what a block hands on: nothing, an output still to add, or a folded input


def fold_between(producer, norm, consumer, ctx: StepContext) -> Optional[tuple]:
    """(norm weight, eps) if the norm between ``producer``'s last product and ``consumer``'s first can be folded
    into the two in this step, else None (parts that do not offer it, other sizes, float32, many rows)."""
    offers = (getattr(producer, "fold_output_weight", None), getattr(norm, "fold", None),
              getattr(consumer, "fold_input_weight", None))
    if None in offers:
        return None
    out_weight, in_weight = offers[0](ctx), offers[2](ctx)
    if out_weight is None or in_weight is None:
        return None
    gated = bool(getattr(consumer, "fold_input_gated", False))
    if not kernels.fold_supported(ctx.n_tokens, ctx.dtype, out_weight, in_weight, gated):
        return None
    return norm.fold()


def adds_into_stream(producer, ctx: StepContext) -> bool:
    """Whether ``producer``'s last product can add its results into the residual stream itself in this step."""
    offer = getattr(producer, "fold_output_weight", None)
    weight = offer(ctx) if offer is not None else None
    return weight is not None and kernels.add_in_product_supported(ctx.n_tokens, ctx.dtype, weight)


@register_block("pre_norm")
class PreNormBlock:
    takes_next_block = True          # forward() has the `next_block` argument and may receive a FoldedInput as `pending`

    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending: Pending, ctx: StepContext, cache: Any,
                next_block: Any = None) -> Pending:
        """``pending`` is the block before's output that is not added yet (None: nothing), or the mixer's input
        already prepared by the block before (its norm folded into the products around it; the residual is up
        to date then).  ``next_block``: the block that runs next, whose first norm this block's feed-forward may
        fold likewise.  Returns what the next block receives as ``pending``."""
        if isinstance(pending, FoldedInput):
            normed = pending
        else:
            normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)
            self.mixer_norm.add_and_norm(residual, pending, normed)
        fold = fold_between(self.mixer, self.feed_forward_norm, self.feed_forward, ctx)
        if fold is not None:
            normed = self.mixer.forward(normed, ctx, cache, fold=NormFold(residual, *fold))
        else:
            if adds_into_stream(self.mixer, ctx):
                delta = self.mixer.forward(normed, ctx, cache, fold=ResidualAdd(residual))      # None: added already
            else:
                delta = self.mixer.forward(normed, ctx, cache)
            normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)      # (the mixer has read the first)
            self.feed_forward_norm.add_and_norm(residual, delta, normed)
        if next_block is not None and getattr(next_block, "takes_next_block", False):
            fold = fold_between(self.feed_forward, getattr(next_block, "mixer_norm", None), getattr(next_block, "mixer", None), ctx)
            if fold is not None:
                return self.feed_forward.forward(normed, ctx, fold=NormFold(residual, *fold))
        if adds_into_stream(self.feed_forward, ctx):
            return self.feed_forward.forward(normed, ctx, fold=ResidualAdd(residual))
        return self.feed_forward.forward(normed, ctx)

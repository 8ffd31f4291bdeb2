"""Interfaces of the part families and their registries.

A *part* is a piece of a layer with its sizes and constants as constructor arguments.  It
declares the tensors it needs by name (:meth:`Part.param_specs`), receives them once they are
on the device (:meth:`Part.load`) and computes on device tensors.  It never learns which model
it is in: whatever it needs arrives as an argument or through the step context.

Families and the signature of their work method:

==============  ==========================================================================
norm            ``add_and_norm(residual, delta, out, rows=None)``: add ``delta`` (or nothing)
                into the float32 residual stream in place, write the norm of the sum to ``out``
position        ``tables(ctx)``: per-step device tables for the rotation; ``fused_args()``
mixer           ``forward(x, ctx, cache) -> y``; ``cache_need()`` says what ``cache`` must be
feed_forward    ``forward(x, ctx) -> y``
block           ``forward(residual, delta, ctx, cache) -> delta``: arranges the four above
==============  ==========================================================================

A new part is a class registered under a name with ``register_norm`` / ``register_position``
/ ``register_mixer`` / ``register_feed_forward`` / ``register_block``; an architecture then
names it in its :class:`~.spec.PartSpec`.

Optional, for speed in steps of few rows: a norm between two matrix products can be *folded* into
them (:class:`NormFold`, :class:`FoldedInput`).  A norm offers it with ``fold()``, a mixer or
feed-forward with ``fold_output_weight(ctx)`` (its last product can add into the residual stream
and prepare the next part's input) and ``fold_input_weight(ctx)`` (its first product can take such
an input); a block uses the fold only where the norm and both neighbours offer it and
``kernels.fold_supported`` agrees, and parts that offer none of this are run as before.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part needs: its name in the checkpoint, its shape and how it is kept.

    ``kind``: ``"matrix"`` is kept in the compute type (bfloat16 or float32); ``"vector"``
    (norm weights and the like) keeps 32 bits if the checkpoint stores 32 bits and takes the
    compute type otherwise; ``"table"`` is an integer table kept as int32.
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class PagedKVNeed:
    """The mixer keeps keys and values per token in pages; ``window`` keys back at most (None: all)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """The mixer keeps one tensor of fixed ``shape`` and ``dtype`` per request (zero at admission)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class NormFold:
    """Handed to a mixer or feed-forward as ``fold=``: instead of returning its output, its last product adds it
    into ``residual`` (float32, in place) and prepares the input of the part behind the norm with ``weight`` and
    ``eps`` (``kernels.linear_residual``).  The part then returns a :class:`FoldedInput`."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float


@dataclass
class ResidualAdd:
    """Handed to a mixer or feed-forward as ``fold=`` where the norm behind it is not folded but the part's last
    product can add its results into ``residual`` (float32, in place) as it stores them
    (``kernels.add_in_product_supported``): the part returns None, and the norm that follows reads the stream
    alone instead of adding a separate output into it first."""

    residual: torch.Tensor


@dataclass
class FoldedInput:
    """What a part receives as ``x`` where the norm before it was folded: ``x = residual * norm weight`` and the
    statistics that its first product completes the norm with (``kernels.RowStats``)."""

    x: torch.Tensor
    stats: Any


class Part:
    """Common base: tensors declared by name, handed over after loading."""

    def param_specs(self) -> list[ParamSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives ``{name: device tensor}`` for exactly the names of :meth:`param_specs`."""


class Registry:
    def __init__(self, family: str) -> None:
        self.family = family
        self._entries: dict[str, Callable[..., Any]] = {}

    def register(self, name: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def decorate(factory: Callable[..., Any]) -> Callable[..., Any]:
            self._entries[name] = factory
            return factory
        return decorate

    def build(self, spec, **context) -> Any:
        try:
            factory = self._entries[spec.kind]
        except KeyError:
            raise KeyError(f"no {self.family} part named {spec.kind!r}; registered: {sorted(self._entries)}") from None
        return factory(**context, **dict(spec.args))

    def names(self) -> list[str]:
        return sorted(self._entries)


NORMS = Registry("norm")
POSITIONS = Registry("position")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed_forward")
BLOCKS = Registry("block")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register

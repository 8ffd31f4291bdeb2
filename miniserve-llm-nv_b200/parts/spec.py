"""Data that describes a model: which parts make up each layer, and in which order layers run.

An architecture module turns its configuration into a :class:`ModelSpec`.  Everything in it
is data: part kinds are registry keys, sizes and constants are arguments, tensor names are
strings.  The model assembled from it (:mod:`.model`) knows no architecture.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by ``kind`` (a key of the registry of its family) with its arguments."""

    kind: str
    args: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward with their norms.

    ``prefix`` is prepended to every tensor name the layer's parts declare.
    """

    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: PartSpec = PartSpec("pre_norm")


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run layer ``layer``.

    ``cache_of`` is ``None`` when the run keeps a cache of its own (if its mixer needs one);
    otherwise it is the index of an earlier entry of the order whose cache this run reads
    without writing to it.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    embedding_name: str
    layers: Sequence[LayerSpec]
    order: Sequence[LayerRun]
    final_norm: PartSpec
    output_name: Optional[str]      # None: the output matrix is the embedding table (tied)
    max_positions: int
    # Names that may be present in a checkpoint without being used (a stored copy of a tied matrix).
    optional_names: Sequence[str] = ()
    # The frame around the layers: embeddings are multiplied by `embedding_scale` as they enter the residual
    # stream; logits are multiplied by `logit_scale` and then, with `logit_softcap` c, become c * tanh(logit / c).
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None

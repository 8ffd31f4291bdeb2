"""The decoder assembled from a :class:`~.spec.ModelSpec`: embedding, the layer runs in the
given order, final norm on the wanted rows, output matrix (with the spec's optional scale of the
embeddings and scale or soft cap of the logits).  It follows the data flow of
miniserve/model/qwen3.py:454-496 and 565-591 but computes logits only for the rows that are
asked for, and knows no architecture: layers, their parts and their order are data.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Union

import torch

from .. import kernels
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PagedKVNeed, ParamSpec, StateNeed
from .context import StepContext
from .spec import ModelSpec


@dataclass(frozen=True)
class CacheGroup:
    """Runs whose caches have the same form share one group (its own pools and page tables)."""

    need: Union[PagedKVNeed, StateNeed]
    n_slots: int          # runs that own a cache in this group


@dataclass(frozen=True)
class RunCache:
    group: int
    slot: int
    writable: bool


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: Union[str, torch.device]) -> None:
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.blocks = []
        for layer in spec.layers:
            mixer = MIXERS.build(layer.mixer, prefix=layer.prefix)
            feed_forward = FEED_FORWARDS.build(layer.feed_forward, prefix=layer.prefix)
            mixer_norm = NORMS.build(layer.mixer_norm, prefix=layer.prefix)
            feed_forward_norm = NORMS.build(layer.feed_forward_norm, prefix=layer.prefix)
            self.blocks.append(BLOCKS.build(layer.block, mixer=mixer, feed_forward=feed_forward,
                                            mixer_norm=mixer_norm, feed_forward_norm=feed_forward_norm))
        self.final_norm = NORMS.build(spec.final_norm)
        for index, run in enumerate(spec.order):
            if not 0 <= run.layer < len(self.blocks):
                raise ValueError(f"order[{index}] names layer {run.layer}, the model has {len(self.blocks)}")
            if run.cache_of is not None and not 0 <= run.cache_of < index:
                raise ValueError(f"order[{index}] reads the cache of entry {run.cache_of}, which does not come before it")
        self.cache_groups, self.run_caches = self._plan_caches()
        self.embedding: Optional[torch.Tensor] = None
        self.output_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ description
    def parts(self):
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm

    def param_specs(self) -> list[ParamSpec]:
        spec = self.spec
        specs = [ParamSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size))]
        for part in self.parts():
            specs.extend(part.param_specs())
        if spec.output_name is not None:
            specs.append(ParamSpec(spec.output_name, (spec.vocab_size, spec.hidden_size)))
        return specs

    def _plan_caches(self) -> tuple[list[CacheGroup], list[Optional[RunCache]]]:
        keys: list[Any] = []
        counts: list[int] = []
        runs: list[Optional[RunCache]] = []
        for index, run in enumerate(self.spec.order):
            mixer = self.blocks[run.layer].mixer
            need = mixer.cache_need() if hasattr(mixer, "cache_need") else None
            if need is None:
                runs.append(None)
                continue
            if run.cache_of is not None:
                source = runs[run.cache_of]
                if source is None or self.cache_groups_need(keys, source.group) != need:
                    raise ValueError(f"order[{index}] cannot read the cache of entry {run.cache_of}: forms differ")
                runs.append(RunCache(source.group, source.slot, writable=False))
                continue
            if need not in keys:
                keys.append(need)
                counts.append(0)
            group = keys.index(need)
            runs.append(RunCache(group, counts[group], writable=True))
            counts[group] += 1
        return [CacheGroup(need, count) for need, count in zip(keys, counts)], runs

    @staticmethod
    def cache_groups_need(keys, group):
        return keys[group]

    # ------------------------------------------------------------------ weights
    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.embedding = tensors[self.spec.embedding_name]
        self.output_weight = self.embedding if self.spec.output_name is None else tensors[self.spec.output_name]
        for part in self.parts():
            part.load({spec.name: tensors[spec.name] for spec in part.param_specs()})

    # ------------------------------------------------------------------ forward
    def forward(self, ctx: StepContext, storage) -> torch.Tensor:
        """Runs the step's tokens through all layer runs; returns float32 logits ``[len(logit_rows), vocab]``."""
        spec = self.spec
        residual = torch.empty((ctx.n_tokens, spec.hidden_size), dtype=torch.float32, device=self.device)
        kernels.embedding(ctx.token_ids, self.embedding, residual, spec.embedding_scale)
        delta = None            # what a block hands to the next: see parts.block
        for index, run in enumerate(spec.order):
            plan = self.run_caches[index]
            cache = None if plan is None else storage.run_view(plan, ctx)
            block = self.blocks[run.layer]
            if getattr(block, "takes_next_block", False):
                following = self.blocks[spec.order[index + 1].layer] if index + 1 < len(spec.order) else None
                delta = block.forward(residual, delta, ctx, cache, following)
            else:
                delta = block.forward(residual, delta, ctx, cache)
        n_rows = ctx.logit_rows.numel()
        logits = torch.empty((n_rows, spec.vocab_size), dtype=torch.float32, device=self.device)
        if n_rows:
            final = torch.empty((n_rows, spec.hidden_size), dtype=self.dtype, device=self.device)
            self.final_norm.add_and_norm(residual, delta, final, rows=ctx.logit_rows)
            kernels.linear(final, self.output_weight, logits)
            if spec.logit_scale != 1.0 or spec.logit_softcap:
                kernels.scale_softcap(logits, spec.logit_scale, spec.logit_softcap)
        return logits

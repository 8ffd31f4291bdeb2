"""Device memory of the cache: page pools per paged group, state tensors per state group, and
the sampling records of the state slots.

A paged group's pools have the shape ``[runs, pages + 1, kv_heads, page_size, head_dim]`` for
keys and the same for values (the layout of miniserve/kv/layout.py:65-75 per group); the last
page is a scratch page that no request ever holds: padding rows of a replayed CUDA graph write
to it.  State tensors and sampling records likewise have one slot more than there are requests,
the scratch slot, which padding rows read and write.  Pools are allocated once and never move.
"""

from __future__ import annotations

import struct
from typing import Sequence

import torch

from ..kernels import SAMPLING_RECORD_WORDS
from ..parts.base import PagedKVNeed, StateNeed
from ..parts.context import PagedKVView, StateView, StepContext
from ..parts.model import CacheGroup, RunCache


class CacheStorage:
    def __init__(self, groups: Sequence[CacheGroup], page_size: int, num_pages: int, max_seqs: int,
                 dtype: torch.dtype, device: torch.device) -> None:
        self.groups = list(groups)
        self.page_size, self.num_pages, self.max_seqs = page_size, num_pages, max_seqs
        self.dtype, self.device = dtype, device
        self.key_pools: list = []
        self.value_pools: list = []
        self.states: list = []
        self.paged_index: list = []     # model group -> index among paged groups (or None)
        paged = 0
        for group in self.groups:
            need = group.need
            if isinstance(need, PagedKVNeed):
                shape = (group.n_slots, num_pages + 1, need.num_kv_heads, page_size, need.head_dim)
                self.key_pools.append(torch.zeros(shape, dtype=dtype, device=device))
                self.value_pools.append(torch.zeros(shape, dtype=dtype, device=device))
                self.states.append(None)
                self.paged_index.append(paged)
                paged += 1
            elif isinstance(need, StateNeed):
                self.key_pools.append(None)
                self.value_pools.append(None)
                self.states.append(torch.zeros((group.n_slots, max_seqs + 1) + tuple(need.shape), dtype=need.dtype,
                                               device=device))
                self.paged_index.append(None)
            else:
                raise TypeError(f"unknown cache need {need!r}")
        self.sampling_records = torch.zeros((max_seqs + 1, SAMPLING_RECORD_WORDS), dtype=torch.int32, device=device)

    @property
    def scratch_page(self) -> int:
        return self.num_pages

    @property
    def scratch_slot(self) -> int:
        """The state slot of padding rows: no request ever holds it."""
        return self.max_seqs

    @staticmethod
    def bytes_per_page(groups: Sequence[CacheGroup], page_size: int, dtype: torch.dtype) -> int:
        """Bytes one page number costs across all paged groups (keys and values, all runs)."""
        size = torch.empty((), dtype=dtype).element_size()
        return sum(2 * g.n_slots * g.need.num_kv_heads * page_size * g.need.head_dim * size
                   for g in groups if isinstance(g.need, PagedKVNeed))

    def run_view(self, plan: RunCache, ctx: StepContext):
        """The cache of one layer run for this step."""
        need = self.groups[plan.group].need
        if isinstance(need, PagedKVNeed):
            block_tables, slots = ctx.group_views[self.paged_index[plan.group]]
            return PagedKVView(self.key_pools[plan.group][plan.slot], self.value_pools[plan.group][plan.slot],
                               block_tables, slots, self.page_size, plan.writable)
        return StateView(self.states[plan.group][plan.slot])

    def reset_slot(self, slot: int, temperature: float, top_p: float, top_k: int, seed: int) -> None:
        """Zeroes the slot's state tensors and writes its sampling record (at admission)."""
        for state in self.states:
            if state is not None:
                state[:, slot].zero_()
        words = struct.unpack("<8i", struct.pack("<ffiIIiii", float(temperature), float(top_p), int(top_k),
                                                 seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, 0, 0, 0))
        self.sampling_records[slot].copy_(torch.tensor(words, dtype=torch.int32), non_blocking=False)

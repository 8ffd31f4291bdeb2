"""What a step hands to the parts: the flat batch and each run's view of its cache.

A step runs ``n_tokens`` tokens of ``n_requests`` requests as one batch.  Request ``r`` owns the
tokens ``query_start[r] .. query_start[r+1]``, which continue its sequence: they sit at the
absolute positions ``context_lens[r] - query_len .. context_lens[r] - 1``.  A request with one
token is a decoded token, one with more a portion of a prompt; the parts treat both alike.
All index tensors are int32 on the device; the ``host_*`` lists carry the same numbers for
parts that loop on the host.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class PagedKVView:
    """One run's keys and values: pools ``[pages, kv_heads, page_size, head_dim]`` of its layer.

    ``block_tables [R, width]`` maps a request's page index to a page of the pool and
    ``slots [N]`` gives each new token's ``page * page_size + offset`` (negative: do not write).
    ``writable`` is False for a run that reads another run's cache.
    """

    key_pool: torch.Tensor
    value_pool: torch.Tensor
    block_tables: torch.Tensor
    slots: torch.Tensor
    page_size: int
    writable: bool = True


@dataclass
class StateView:
    """One run's fixed-size state: ``states[slot]`` belongs to the request in that state slot."""

    states: torch.Tensor


@dataclass
class StepContext:
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    request_of_token: torch.Tensor
    query_start: torch.Tensor
    context_lens: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    max_query_len: int
    max_context_len: int
    dtype: torch.dtype
    device: torch.device
    host_query_start: list[int] = field(default_factory=list)
    host_context_lens: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    memo: dict[Any, Any] = field(default_factory=dict)   # per-step scratch shared by parts (rotation tables)
    group_views: list[Any] = field(default_factory=list)  # per cache group: (block_tables, slots)

    def buffer(self, name: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """An uninitialised device tensor for a part's intermediate result, the same one for every call of a step
        with the same name, shape and type.  The layers of a step run one after the other on one stream, so a
        layer's intermediates can live where the layer before kept its own; a step of 28 layers then allocates
        nine tensors, not 250 (an allocation costs the host more than some kernels cost the device).  A tensor
        that outlives the step (the logits) must not come from here."""
        key = ("buffer", name, shape, dtype)
        found = self.memo.get(key)
        if found is None:
            found = self.memo[key] = torch.empty(shape, dtype=dtype, device=self.device)
        return found

"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step's entries may be portions of prompts of any length beside single decoded tokens.  They
are flattened into one batch (no padding), every index a kernel will use is checked on the
host (miniserve/engine/flat_batch.py:490-569 does the same for its decode rows), the index
arrays travel to the device in one copy, the model runs once over all tokens, and the logits
come back only for the positions that were asked for.  MiniServe runs a step as one forward
per prompt portion plus one for the decode rows (miniserve/engine/executor.py:239-255) and
computes logits for every position of a portion; this engine does neither.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..cache.manager import RELEASED, CacheManager, StepReservation
from ..parts.context import StepContext


@dataclass
class StepEntry:
    """A request's next tokens and the indices among them whose logits are wanted."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


class StepFunction:
    def __init__(self, model, storage, manager: CacheManager, max_model_len: int) -> None:
        self.model, self.storage, self.manager = model, storage, manager
        self.max_model_len = max_model_len
        self.device = model.device
        self.vocab_size = model.spec.vocab_size
        self.launches = 0            # steps run (for the bench's bookkeeping)

    # ------------------------------------------------------------------ batch building
    def build_context(self, entries: Sequence[StepEntry], reservation: StepReservation) -> StepContext:
        manager, ps = self.manager, self.manager.page_size
        if len(entries) != len(reservation.items):
            raise ValueError("the reservation was made for other entries")
        tokens: list[int] = []
        positions: list[int] = []
        request_of_token: list[int] = []
        query_start = [0]
        context_lens: list[int] = []
        state_slots: list[int] = []
        logit_rows: list[int] = []
        n_groups = len(manager.paged_needs)
        slots: list[list[int]] = [[] for _ in range(n_groups)]
        width = 1
        for row, (entry, item) in enumerate(zip(entries, reservation.items)):
            if entry.request_id != item.request_id or len(entry.tokens) != item.end - item.start:
                raise ValueError(f"entry {row} does not match its reservation")
            if item.end > self.max_model_len:
                raise ValueError(f"request {entry.request_id!r} would reach {item.end} tokens; the limit is {self.max_model_len}")
            for token in entry.tokens:
                if not 0 <= int(token) < self.vocab_size:
                    raise ValueError(f"token id {token} outside the vocabulary of {self.vocab_size}")
            base = len(tokens)
            for index in entry.want:
                if not 0 <= index < len(entry.tokens):
                    raise ValueError(f"wanted index {index} outside the {len(entry.tokens)} tokens of the entry")
                logit_rows.append(base + index)
            tokens.extend(int(t) for t in entry.tokens)
            positions.extend(range(item.start, item.end))
            request_of_token.extend([row] * len(entry.tokens))
            query_start.append(len(tokens))
            context_lens.append(item.end)
            state_slots.append(manager.requests[entry.request_id].slot)
            for group in range(n_groups):
                slots[group].extend(item.slots[group])
                width = max(width, len(item.tables[group]))

        scratch = self.storage.scratch_page
        limit = self.storage.num_pages
        tables: list[list[int]] = []
        for group in range(n_groups):
            flat: list[int] = []
            for item in reservation.items:
                table = item.tables[group]
                for page in table:
                    if page != RELEASED and not 0 <= page < limit:
                        raise ValueError(f"page {page} outside the pool of {limit}")
                flat.extend(scratch if page == RELEASED else page for page in table)
                flat.extend([scratch] * (width - len(table)))
            tables.append(flat)
            for slot in slots[group]:
                if not 0 <= slot < limit * ps:
                    raise ValueError(f"slot {slot} outside the pool")

        n, r = len(tokens), len(entries)
        pieces = [tokens, positions, request_of_token, query_start, context_lens, state_slots, logit_rows]
        for group in range(n_groups):
            pieces += [tables[group], slots[group]]
        total = sum(len(p) for p in pieces)
        staging = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        offset = 0
        spans = []
        for piece in pieces:
            if piece:
                staging[offset:offset + len(piece)] = torch.tensor(piece, dtype=torch.int32)
            spans.append((offset, len(piece)))
            offset += len(piece)
        on_device = staging.to(self.device, non_blocking=True)
        views = [on_device[start:start + length] for start, length in spans]
        group_views = []
        for group in range(n_groups):
            group_views.append((views[7 + 2 * group].view(r, width), views[8 + 2 * group]))
        return StepContext(
            n_tokens=n, n_requests=r, token_ids=views[0], positions=views[1], request_of_token=views[2],
            query_start=views[3], context_lens=views[4], state_slots=views[5], logit_rows=views[6],
            max_query_len=max((len(e.tokens) for e in entries), default=0),
            max_context_len=max(context_lens, default=0), dtype=self.model.dtype, device=self.device,
            host_query_start=query_start, host_context_lens=context_lens, host_state_slots=state_slots,
            group_views=group_views)

    # ------------------------------------------------------------------ running
    def run(self, entries: Sequence[StepEntry], reservation: StepReservation) -> torch.Tensor:
        """float32 logits ``[number of wanted positions, vocab]`` on the device, in entry order."""
        ctx = self.build_context(entries, reservation)
        self.launches += 1
        return self.model.forward(ctx, self.storage)

"""The scheduler: which requests run how many tokens in the next step.

Policy of miniserve/engine/scheduler.py:129-227: requests in order of arrival (ties by id);
decoding requests first, one token each; then prompt portions, cut to the remaining token
budget (and to ``prefill_chunk_size``) when chunked prefill is on; nothing is planned that the
free pages (plus the reusable prefixes that could be evicted) cannot hold; a waiting request
is admitted only while a state slot is free.  When chunked prefill is on and some prompt can
make progress, one sequence and one token of the budget are kept back for it so that decodes
cannot starve prompts.

What it adds: MiniServe plans nothing for a request that does not fit and can stall for good
when running requests hold all pages between them.  Here, if no running request can make
progress, :meth:`choose_victim` names the youngest running request, which the engine preempts
(its pages are given back; it is recomputed later), so that the oldest request always finishes.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence as Seq

from ..cache.manager import CapacitySnapshot
from .sequence import Sequence, Status


@dataclass(frozen=True)
class PlanItem:
    request_id: str
    start: int
    end: int
    is_decode: bool


@dataclass(frozen=True)
class StepPlan:
    step_id: int
    items: tuple[PlanItem, ...]
    scheduled_tokens: int

    @property
    def is_empty(self) -> bool:
        return not self.items


class Scheduler:
    def __init__(self, *, max_num_seqs: int, max_num_batched_tokens: int, enable_chunked_prefill: bool = True,
                 prefill_chunk_size: Optional[int] = None) -> None:
        if max_num_seqs < 1 or max_num_batched_tokens < 1:
            raise ValueError("the scheduler needs at least one sequence and one token per step")
        if prefill_chunk_size is not None and (prefill_chunk_size < 1 or not enable_chunked_prefill
                                               or prefill_chunk_size > max_num_batched_tokens):
            raise ValueError("prefill_chunk_size needs chunked prefill and must lie within the token budget")
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.enable_chunked_prefill = enable_chunked_prefill
        self.prefill_chunk_size = prefill_chunk_size
        self._next_step = 0

    def repeat_decode_plan(self, rows: Seq[tuple[str, int, int]]) -> StepPlan:
        """The plan of a step that decodes the same requests as the step before: (request, start, end) each."""
        step_id = self._next_step
        self._next_step += 1
        return StepPlan(step_id, tuple(PlanItem(r, start, end, True) for r, start, end in rows), len(rows))

    @staticmethod
    def _take(available: list[int], need: Seq[int]) -> bool:
        """Takes ``need`` pages per group out of ``available`` if every group has them."""
        if any(n > a for n, a in zip(need, available)):
            return False
        for group, n in enumerate(need):
            available[group] -= n
        return True

    def schedule(self, sequences: Seq[Sequence], capacity: CapacitySnapshot) -> StepPlan:
        step_id = self._next_step
        self._next_step += 1
        ordered = sorted((s for s in sequences if not s.done), key=lambda s: (s.arrival, s.request_id))
        token_budget = self.max_num_batched_tokens
        seq_budget = self.max_num_seqs
        available = capacity.available()        # pages per cache group; the cache says what a portion needs of each
        free_slots = capacity.free_slots
        items: list[PlanItem] = []

        prompts = [s for s in ordered if not s.is_decoding]
        progressable = any(s.status is Status.RUNNING or free_slots > 0 for s in prompts)
        reserve = 1 if self.enable_chunked_prefill and progressable else 0

        for seq in ordered:
            if not seq.is_decoding:
                continue
            if seq_budget <= reserve or token_budget <= reserve:
                break
            if not self._take(available, capacity.pages_for(seq.computed, seq.computed + 1)):
                continue
            items.append(PlanItem(seq.request_id, seq.computed, seq.computed + 1, True))
            seq_budget -= 1
            token_budget -= 1

        for seq in prompts:
            if seq_budget == 0 or token_budget == 0:
                break
            if seq.status is Status.WAITING:
                if free_slots == 0:
                    continue
            take = min(seq.remaining, token_budget) if self.enable_chunked_prefill else seq.remaining
            if self.prefill_chunk_size is not None:
                take = min(take, self.prefill_chunk_size)
            if take <= 0 or take > token_budget:
                continue
            if not self._take(available, capacity.pages_for(seq.computed, seq.computed + take)):
                if not self.enable_chunked_prefill:
                    continue
                take = min(take, capacity.room(seq.computed, available))      # the longest portion the pages can hold
                if take <= 0 or not self._take(available, capacity.pages_for(seq.computed, seq.computed + take)):
                    continue
            items.append(PlanItem(seq.request_id, seq.computed, seq.computed + take, False))
            if seq.status is Status.WAITING:
                free_slots -= 1
            seq_budget -= 1
            token_budget -= take

        return StepPlan(step_id, tuple(items), self.max_num_batched_tokens - token_budget)

    @staticmethod
    def choose_victim(sequences: Seq[Sequence]) -> Optional[Sequence]:
        """The running request to preempt when nothing can make progress: the youngest that holds pages."""
        running = [s for s in sequences if s.status is Status.RUNNING and s.computed > 0]
        if len(running) < 2:
            return None
        return max(running, key=lambda s: (s.arrival, s.request_id))

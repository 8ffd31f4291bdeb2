"""The engine loop: admit, plan, reserve, run, sample, commit, finish and free.

With ``look_ahead`` (and an executor that can defer reading a step's tokens) decoding runs one step
ahead of the host: a step of decoded tokens is started and its tokens are read only during the next
call, after that call has started the following step, whose input tokens the device takes from the
sampled ones directly.  The host's work for a step then overlaps the device's work for the step before.
A request that ends on a stop token is found one step late; the extra token computed for it is dropped
with its pages.  Whenever the next step would not be the same rows again (a request reaches its token
budget, another waits or is part-way through its prompt, pages run short), the pending tokens are read
first and the step is planned as usual.

One call of :meth:`Engine.step` is one transaction, in the order of
miniserve/engine/core.py:278-439: finished requests give back what they hold; the scheduler
plans; newly planned requests are admitted to the cache (a state slot, reusable prefix pages);
the cache manager reserves pages; the executor runs the batch and samples; then the cache, the
sequences and the prefix cache are updated.  If anything raises before the commit, the
reservation is aborted, so pages and lengths are as before the step, and the requests of that
step are failed (core.py:365-434).
"""

from __future__ import annotations

import secrets
import time
from dataclasses import dataclass, field
from typing import Optional, Protocol, Sequence as Seq

from ..cache.allocator import OutOfPagesError
from ..cache.manager import CacheManager, StepReservation
from ..sampling.params import SamplingParams
from .scheduler import Scheduler, StepPlan
from .sequence import Sequence, Status
from .step import StepEntry


@dataclass
class SampleRequest:
    """One row to sample: the entry it ends, the request's state slot and its draw index."""

    entry: int
    slot: int
    draw_index: int


class Executor(Protocol):
    """``execute`` is required; an executor may also offer ``can_defer(entries)`` and
    ``execute_deferred(entries, reservation, samples, feed_back)`` returning an object whose ``tokens()``
    waits for the step's tokens, which the engine's look-ahead uses."""

    def admit(self, slot: int, params: SamplingParams, seed: int) -> None: ...

    def execute(self, entries: Seq[StepEntry], reservation: StepReservation,
                samples: Seq[SampleRequest]) -> list[int]: ...


@dataclass
class GenerationResult:
    request_id: str
    token_ids: list[int]
    finish_reason: Optional[str]
    prompt_len: int = 0
    preemptions: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    empty_steps: int = 0
    scheduled_tokens: int = 0
    decode_tokens: int = 0
    prefill_tokens: int = 0
    preemptions: int = 0
    prefix_hit_tokens: int = 0
    failed_steps: int = 0


class RequestRejected(ValueError):
    """The request cannot be accepted; the message says which limit it breaks."""


class Engine:
    def __init__(self, manager: CacheManager, scheduler: Scheduler, executor: Executor, *, vocab_size: int,
                 max_model_len: int, max_pending_requests: int = 64, look_ahead: bool = False) -> None:
        self.manager, self.scheduler, self.executor = manager, scheduler, executor
        self.look_ahead = look_ahead and hasattr(executor, "execute_deferred")
        self._pending: Optional[tuple[list[Sequence], object]] = None    # a started step whose tokens are unread
        self.vocab_size, self.max_model_len = vocab_size, max_model_len
        self.max_pending_requests = max_pending_requests
        self.sequences: dict[str, Sequence] = {}
        self.finished: dict[str, GenerationResult] = {}
        self.stats = EngineStats()
        self.last_plan: Optional[StepPlan] = None
        self.last_step_ran = False
        self._arrivals = 0

    # ------------------------------------------------------------------ admission
    def submit(self, request_id: str, prompt: Seq[int], params: SamplingParams, arrival: Optional[int] = None) -> None:
        """Checks of miniserve/engine/core.py:193-265."""
        if request_id in self.sequences or request_id in self.finished:
            raise RequestRejected(f"duplicate request id {request_id!r}")
        if len(self.sequences) >= self.max_pending_requests:
            raise RequestRejected(f"MAX_PENDING_REQUESTS: {self.max_pending_requests} requests are already pending")
        prompt = tuple(int(t) for t in prompt)
        if not prompt:
            raise RequestRejected("the prompt must hold at least one token")
        if len(prompt) + params.max_new_tokens > self.max_model_len:
            raise RequestRejected(f"prompt ({len(prompt)}) plus max_new_tokens ({params.max_new_tokens}) exceeds "
                                  f"max_model_len ({self.max_model_len})")
        page_size = self.manager.page_size
        if (len(prompt) + params.max_new_tokens + page_size - 1) // page_size > self.manager.num_pages:
            raise RequestRejected("CONTEXT_CAPACITY_EXCEEDED: the request alone needs more pages than the pool has")
        if any(not 0 <= t < self.vocab_size for t in prompt) or any(t >= self.vocab_size for t in params.stop_token_ids):
            raise RequestRejected(f"a token id lies outside the vocabulary of {self.vocab_size}")
        if params.top_k > self.vocab_size:
            raise RequestRejected("top_k exceeds the vocabulary size")
        if not self.scheduler.enable_chunked_prefill and len(prompt) > self.scheduler.max_num_batched_tokens:
            raise RequestRejected("CHUNKED_PREFILL_DISABLED: the prompt exceeds max_num_batched_tokens")
        if arrival is None:
            arrival = self._arrivals
        self._arrivals = max(self._arrivals, arrival) + 1
        seed = params.seed if params.seed is not None else secrets.randbits(63)
        self.sequences[request_id] = Sequence(request_id, prompt, params, arrival, seed)

    # ------------------------------------------------------------------ one step
    def _finalize(self) -> None:
        for request_id, seq in list(self.sequences.items()):
            if not seq.done:
                continue
            if request_id in self.manager.requests:
                self.manager.release(request_id)
            self.finished[request_id] = GenerationResult(request_id, list(seq.generated), seq.finish_reason,
                                                         len(seq.prompt), seq.preemptions)
            del self.sequences[request_id]

    def _preempt(self, seq: Sequence) -> None:
        self.manager.release(seq.request_id)
        seq.preempt()
        self.stats.preemptions += 1

    # ------------------------------------------------------------------ decoding one step ahead
    def _read_pending(self) -> None:
        """Reads the tokens of the started step and gives them to their sequences."""
        sequences, handle = self._pending
        self._pending = None
        for seq, token in zip(sequences, handle.tokens()):
            if not seq.done:
                seq.append_sampled(token)

    def _step_ahead(self) -> Optional[StepPlan]:
        """Starts the step after the pending one if it is the same rows again, then reads the pending
        tokens; None if the next step has to be planned in the usual way."""
        sequences, _ = self._pending
        if any(s.done or len(s.generated) + 2 > s.params.max_new_tokens for s in sequences):
            return None                      # a row ends with the pending token: the rows change
        if len(sequences) != len(self.sequences):
            return None                      # another request waits or is part-way through its prompt
        try:
            reservation = self.manager.prepare([(s.request_id, 1) for s in sequences])
        except OutOfPagesError:
            return None
        # the pending token of a row is token number `total` of its sequence; its value is still on the device
        entries = [StepEntry(s.request_id, [0], [0]) for s in sequences]
        samples = [SampleRequest(i, self.manager.requests[s.request_id].slot, len(s.generated) + 1)
                   for i, s in enumerate(sequences)]
        try:
            handle = self.executor.execute_deferred(entries, reservation, samples, feed_back=True)
        except BaseException as error:
            # as in an ordinary step: pages and lengths as before it, its requests failed; the tokens of the
            # step before are still read
            self.manager.abort(reservation)
            self.stats.failed_steps += 1
            self._read_pending()
            for seq in sequences:
                if not seq.done:
                    seq.finish(f"error: {type(error).__name__}", failed=True)
            if isinstance(error, Exception):
                self._finalize()
            raise
        self.manager.commit(reservation)
        self._read_pending()                 # the device is busy with the new step meanwhile
        running = []
        for seq in sequences:
            if not seq.done:                 # (a stop token ended it: the step just started has a row to drop)
                seq.advance(seq.total)
                self.stats.decode_tokens += 1
                self.stats.scheduled_tokens += 1
            running.append(seq)
        self._pending = (running, handle)
        self.stats.steps += 1
        self.last_step_ran = True
        self.last_plan = plan = self.scheduler.repeat_decode_plan([(r.request_id, r.start, r.end)
                                                                   for r in reservation.items])
        self._finalize()
        return plan

    def step(self) -> StepPlan:
        if self._pending is not None:
            plan = self._step_ahead()
            if plan is not None:
                return plan
            self._read_pending()
        self._finalize()
        live = list(self.sequences.values())
        plan = self.scheduler.schedule(live, self.manager.capacity())
        while plan.is_empty and live:
            victim = self.scheduler.choose_victim(live)
            if victim is None:
                break
            self._preempt(victim)
            plan = self.scheduler.schedule(live, self.manager.capacity())
        self.last_plan = plan
        self.last_step_ran = False
        self.stats.steps += 1
        if plan.is_empty:
            self.stats.empty_steps += 1
            return plan

        # admit newly planned requests; a reusable prefix may move the start of their portion
        items = []
        admitted_now = set()
        for item in plan.items:
            seq = self.sequences[item.request_id]
            start, end = item.start, item.end
            if seq.status is Status.WAITING:
                entry = self.manager.admit(seq.request_id)
                self.executor.admit(entry.slot, seq.params, seq.seed)
                seq.status = Status.RUNNING
                admitted_now.add(seq.request_id)
                matched = self.manager.attach_prefix(seq.request_id, seq.tokens)
                if matched:
                    seq.computed = matched
                    self.stats.prefix_hit_tokens += matched
                    start, end = matched, min(seq.total, max(item.end, matched + 1))
            items.append((seq, start, end, item.is_decode))

        # The plan rests on an estimate of free pages.  If the reservation does not fit after all,
        # the last planned (youngest, lowest priority) request waits for a later step.
        reservation = None
        while items:
            try:
                reservation = self.manager.prepare([(seq.request_id, end - start) for seq, start, end, _ in items])
                break
            except OutOfPagesError:
                self.stats.failed_steps += 1
                dropped = items.pop()[0]
                if dropped.request_id in admitted_now:
                    # back out of the admission too: reusable pages it pinned can be evicted for older requests
                    self.manager.release(dropped.request_id)
                    dropped.status, dropped.computed = Status.WAITING, 0
        if reservation is None:
            victim = self.scheduler.choose_victim(live)
            if victim is not None:
                self._preempt(victim)
            return plan
        entries = [StepEntry(seq.request_id, seq.token_slice(start, end), [end - start - 1] if end == seq.total else [])
                   for seq, start, end, _ in items]
        samples = [SampleRequest(index, self.manager.requests[seq.request_id].slot, len(seq.generated))
                   for index, (seq, start, end, _) in enumerate(items) if end == seq.total]
        defer = (self.look_ahead and len(samples) == len(entries) and all(d for *_, d in items)
                 and self.executor.can_defer(entries))
        try:
            if defer:
                handle = self.executor.execute_deferred(entries, reservation, samples)
                tokens = []
            else:
                tokens = self.executor.execute(entries, reservation, samples)
        except BaseException as error:
            self.manager.abort(reservation)
            self.stats.failed_steps += 1
            for seq, *_ in items:
                seq.finish(f"error: {type(error).__name__}", failed=True)
            if not isinstance(error, Exception):
                raise
            self._finalize()
            raise
        self.manager.commit(reservation)
        self.last_step_ran = True

        for seq, start, end, is_decode in items:
            seq.advance(end)
            if is_decode:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += end - start
        if defer:
            self._pending = ([seq for seq, *_ in items], handle)
        for sample, token in zip(samples, tokens):
            items[sample.entry][0].append_sampled(token)
        for seq, *_ in items:
            if not seq.prompt_cached and seq.computed >= len(seq.prompt):
                self.manager.cache_prefix(seq.request_id, seq.prompt)
                seq.prompt_cached = True
        self.stats.scheduled_tokens += sum(end - start for _, start, end, _ in items)
        self._finalize()
        return plan

    # ------------------------------------------------------------------ driving
    def has_unfinished(self) -> bool:
        return self._pending is not None or any(not s.done for s in self.sequences.values())

    def run_until_done(self, max_steps: int = 1_000_000) -> None:
        stalled = 0
        for _ in range(max_steps):
            if not self.has_unfinished():
                break
            self.step()
            stalled = 0 if self.last_step_ran else stalled + 1
            if stalled > 8:
                raise RuntimeError("the scheduler cannot make progress: no request fits the free pages and state slots")
        if self._pending is not None:
            self._read_pending()
        self._finalize()

    def take_result(self, request_id: str) -> GenerationResult:
        return self.finished.pop(request_id)

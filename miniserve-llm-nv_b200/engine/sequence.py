"""A request's token state.

A sequence is its prompt followed by what it has generated; ``computed`` counts the tokens
whose keys and values are committed to the cache.  Running the last uncomputed token yields
the logits from which the next token is sampled, so while a sequence decodes exactly one
token is pending: ``len(tokens) == computed + 1`` (the invariant of
miniserve/engine/state.py:41-43).  Prompt portions and decoded tokens are the same thing here:
a step runs ``tokens[computed:computed + n]`` and samples only when it reaches the end.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional

import numpy

from ..sampling.params import SamplingParams


class Status(enum.Enum):
    WAITING = "waiting"          # holds nothing in the cache (new, or preempted)
    RUNNING = "running"          # admitted: has a state slot, maybe pages
    FINISHED = "finished"
    FAILED = "failed"


@dataclass
class Sequence:
    request_id: str
    prompt: tuple[int, ...]
    params: SamplingParams
    arrival: int
    seed: int
    generated: list[int] = field(default_factory=list)
    computed: int = 0
    status: Status = Status.WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0
    prompt_cached: bool = False      # its prompt pages were offered for reuse
    _prompt_array: Optional[numpy.ndarray] = field(default=None, repr=False, compare=False)

    @property
    def tokens(self) -> list[int]:
        return list(self.prompt) + self.generated

    @property
    def total(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def remaining(self) -> int:
        return self.total - self.computed

    @property
    def is_decoding(self) -> bool:
        return self.status is Status.RUNNING and self.remaining == 1 and self.computed > 0 and bool(self.generated)

    @property
    def done(self) -> bool:
        return self.status in (Status.FINISHED, Status.FAILED)

    def token_slice(self, start: int, end: int):
        """Tokens ``start .. end - 1``: a view of the prompt held as an int64 array where the slice lies within the
        prompt (a portion of thousands of tokens is then handed to the step without being rebuilt number by number),
        else a list."""
        n_prompt = len(self.prompt)
        if end <= n_prompt:
            if self._prompt_array is None:
                self._prompt_array = numpy.asarray(self.prompt, dtype=numpy.int64)
            return self._prompt_array[start:end]
        return (list(self.prompt[start:]) if start < n_prompt else []) + self.generated[max(start - n_prompt, 0):end - n_prompt]

    def advance(self, end: int) -> None:
        if not self.computed < end <= self.total:
            raise RuntimeError(f"{self.request_id}: cannot advance from {self.computed} to {end} of {self.total}")
        self.computed = end

    def append_sampled(self, token: int) -> None:
        """Adds the token sampled at the end of the sequence and decides whether it ends there
        (miniserve/engine/state.py:148-166: a stop token ends with "stop", the token budget with "length")."""
        if self.remaining != 0:
            raise RuntimeError(f"{self.request_id}: sampled before the sequence was computed to its end")
        self.generated.append(int(token))
        if int(token) in self.params.stop_token_ids:
            self.finish("stop")
        elif len(self.generated) >= self.params.max_new_tokens:
            self.finish("length")

    def finish(self, reason: str, failed: bool = False) -> None:
        self.status = Status.FAILED if failed else Status.FINISHED
        self.finish_reason = reason

    def preempt(self) -> None:
        """Back to waiting with nothing in the cache; what was generated is kept and recomputed."""
        self.status = Status.WAITING
        self.computed = 0
        self.preemptions += 1

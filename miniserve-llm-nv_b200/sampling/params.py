"""Sampling parameters of a request, with MiniServe's names, meanings and bounds
(miniserve/engine/request.py:9-59)."""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class SamplingParams:
    """``temperature == 0`` is greedy; otherwise temperature, then top-k, then top-p, then a draw.

    ``top_k == 0`` and ``top_p == 1`` switch those filters off.  ``seed`` fixes the request's
    random stream (``None``: a fresh one); the stream belongs to the request alone, so what
    else is in a batch never changes what is drawn.
    """

    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    max_new_tokens: int = 4
    stop_token_ids: tuple[int, ...] = ()
    seed: Optional[int] = None

    def __post_init__(self) -> None:
        t = self.temperature
        if not isinstance(t, (int, float)) or isinstance(t, bool) or not math.isfinite(t) or not 0 <= t <= 2:
            raise ValueError("temperature must be finite and in [0, 2].")
        p = self.top_p
        if not isinstance(p, (int, float)) or isinstance(p, bool) or not math.isfinite(p) or not 0 < p <= 1:
            raise ValueError("top_p must be in (0, 1].")
        if not isinstance(self.top_k, int) or isinstance(self.top_k, bool) or self.top_k < 0:
            raise ValueError("top_k must be non-negative.")
        if not isinstance(self.max_new_tokens, int) or isinstance(self.max_new_tokens, bool) or self.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive.")
        if not isinstance(self.stop_token_ids, tuple):
            raise ValueError("stop_token_ids must be an immutable tuple.")
        if any(not isinstance(t, int) or isinstance(t, bool) or t < 0 for t in self.stop_token_ids):
            raise ValueError("stop_token_ids must contain non-negative integers.")
        if len(set(self.stop_token_ids)) != len(self.stop_token_ids):
            raise ValueError("stop_token_ids must not contain duplicates.")
        if self.seed is not None and (not isinstance(self.seed, int) or isinstance(self.seed, bool)
                                      or not 0 <= self.seed <= 2 ** 63 - 1):
            raise ValueError("seed must be an integer in [0, 2^63-1] or None.")

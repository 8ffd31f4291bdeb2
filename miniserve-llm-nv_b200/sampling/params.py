"""Sampling parameters of a request.  Field names, defaults and bounds are MiniServe's
(miniserve/engine/request.py:9-59), so that a request written for it means the same here."""

from __future__ import annotations

import math
from dataclasses import dataclass, fields
from typing import Optional

MAX_SEED = 2 ** 63 - 1


def _whole(name: str, value, low: int, high: Optional[int] = None) -> None:
    """An integer field (a bool is not one) within ``low .. high``."""
    if not isinstance(value, int) or isinstance(value, bool) or value < low or (high is not None and value > high):
        upper = "" if high is None else f" and at most {high}"
        raise ValueError(f"{name}={value!r}: expected an integer of at least {low}{upper}")


def _real(name: str, value, low: float, high: float, low_open: bool = False) -> None:
    """A finite number (a bool is not one) within ``low .. high``; ``low_open`` leaves ``low`` itself out."""
    ok = (isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)
          and low <= value <= high and not (low_open and value == low))
    if not ok:
        left = "(" if low_open else "["
        raise ValueError(f"{name}={value!r}: expected a finite number in {left}{low:g}, {high:g}]")


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
        _real("temperature", self.temperature, 0.0, 2.0)
        _real("top_p", self.top_p, 0.0, 1.0, low_open=True)
        _whole("top_k", self.top_k, 0)
        _whole("max_new_tokens", self.max_new_tokens, 1)
        if self.seed is not None:
            _whole("seed", self.seed, 0, MAX_SEED)
        stops = self.stop_token_ids
        if not isinstance(stops, tuple):
            raise ValueError(f"stop_token_ids={stops!r}: expected a tuple (the parameters are immutable)")
        for index, token in enumerate(stops):
            _whole(f"stop_token_ids[{index}]", token, 0)
        if len(set(stops)) != len(stops):
            repeated = sorted({t for t in stops if stops.count(t) > 1})
            raise ValueError(f"stop_token_ids names {repeated} more than once")

    def describe(self) -> str:
        """``name=value`` of every field that differs from its default (for logs and error messages)."""
        changed = [f"{f.name}={getattr(self, f.name)!r}" for f in fields(self) if getattr(self, f.name) != f.default]
        return ", ".join(changed) or "defaults"

"""Runs a planned step on the device: the step function, then the sampling kernel, then one
device-to-host copy of the chosen tokens (MiniServe reads one token per request per step:
miniserve/model/sampling.py:151,174,208)."""

from __future__ import annotations

from typing import Sequence as Seq

import torch

from .. import kernels
from ..cache.manager import StepReservation
from ..sampling.params import SamplingParams
from .step import StepEntry, StepFunction


class PendingTokens:
    """The tokens of a step that may still be running: :meth:`tokens` waits for them."""

    def __init__(self, buffer: torch.Tensor, count: int, ready: "torch.cuda.Event") -> None:
        self.buffer, self.count, self.ready = buffer, count, ready

    def tokens(self) -> list[int]:
        self.ready.synchronize()
        return self.buffer[:self.count].tolist()


class DeviceExecutor:
    def __init__(self, step_function: StepFunction, storage) -> None:
        self.step_function, self.storage = step_function, storage
        self.device = step_function.device
        self._token_buffers: list[torch.Tensor] = []      # two pinned buffers, used in turn
        self._turn = 0

    def can_defer(self, entries: Seq[StepEntry]) -> bool:
        """Whether :meth:`execute_deferred` takes these entries (a replayed step of single tokens)."""
        return self.step_function.replays(entries)

    def execute_deferred(self, entries: Seq[StepEntry], reservation: StepReservation, samples,
                         feed_back: bool = False) -> PendingTokens:
        """Starts the step and returns at once; the tokens are read later.  ``feed_back``: every row's
        token is the one that the step before sampled for it (same rows, same order), taken on the device."""
        if len(samples) != len(entries):
            raise ValueError("a deferred step samples every row")
        self.step_function.run(entries, reservation, [s.draw_index for s in samples], feed_back=feed_back)
        chosen = self.step_function.last_tokens
        if not self._token_buffers:
            rows = max(self.step_function.graphs)
            self._token_buffers = [torch.empty(rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        if self._token_buffers[0].numel() < len(entries):
            self._token_buffers = [torch.empty(len(entries), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        buffer = self._token_buffers[self._turn]
        self._turn ^= 1
        buffer[:len(entries)].copy_(chosen, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record()
        return PendingTokens(buffer, len(entries), ready)

    def admit(self, slot: int, params: SamplingParams, seed: int) -> None:
        self.storage.reset_slot(slot, params.temperature, params.top_p, params.top_k, seed)

    def execute(self, entries: Seq[StepEntry], reservation: StepReservation, samples) -> list[int]:
        draws = None
        if len(samples) == len(entries):
            draws = [s.draw_index for s in samples]
        logits = self.step_function.run(entries, reservation, draws)
        if not samples:
            return []
        if self.step_function.last_tokens is not None:      # a replayed graph sampled already
            return self.step_function.last_tokens.cpu().tolist()
        # an eager step may have run kernels with bounded waits (the tcgen05 attention of prompt portions)
        kernels.check_device_errors(self.device)
        meta = torch.tensor([[s.slot for s in samples], [s.draw_index for s in samples]], dtype=torch.int32,
                            pin_memory=self.device.type == "cuda").to(self.device, non_blocking=True)
        chosen = torch.empty(len(samples), dtype=torch.int32, device=self.device)
        kernels.sample(logits, self.storage.sampling_records, meta[0], meta[1], chosen)
        return chosen.cpu().tolist()

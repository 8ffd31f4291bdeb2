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


class DeviceExecutor:
    def __init__(self, step_function: StepFunction, storage) -> None:
        self.step_function, self.storage = step_function, storage
        self.device = step_function.device

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

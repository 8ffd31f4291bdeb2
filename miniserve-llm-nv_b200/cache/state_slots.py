"""Slots for per-request state of fixed size.

Every live request holds one slot from admission to release.  A slot indexes the device
records that belong to the request: its sampling record (temperature, top-p, top-k and the
seed of its random stream) and, for each state group of the model, one tensor of the group's
fixed shape (zeroed at admission).  The Qwen3 dense decoder has no state group; the sampling
record is what its requests keep here.
"""

from __future__ import annotations

import heapq


class OutOfSlotsError(RuntimeError):
    """All state slots are held by live requests."""


class StateSlots:
    def __init__(self, num_slots: int) -> None:
        if num_slots < 1:
            raise ValueError("at least one state slot is needed")
        self.num_slots = num_slots
        self._free = list(range(num_slots))
        self._owner: dict[int, str] = {}

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self, owner: str) -> int:
        if not self._free:
            raise OutOfSlotsError(f"OUT_OF_SLOTS: all {self.num_slots} state slots are in use")
        slot = heapq.heappop(self._free)
        self._owner[slot] = owner
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._owner:
            raise RuntimeError(f"state slot {slot} is freed twice")
        del self._owner[slot]
        heapq.heappush(self._free, slot)

    def owner(self, slot: int):
        return self._owner.get(slot)

    def check_invariants(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free) or free & set(self._owner) or len(free) + len(self._owner) != self.num_slots:
            raise AssertionError("state slots: free list and owners disagree")

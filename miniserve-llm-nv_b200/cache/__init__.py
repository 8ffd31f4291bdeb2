"""Paged key/value cache: allocator, block tables, state slots, prefix reuse, device pools."""

from .allocator import OutOfPagesError, PageAllocator
from .manager import RELEASED, CacheManager, CapacitySnapshot, ReservedItem, RequestCache, StepReservation
from .prefix import PrefixCache
from .state_slots import OutOfSlotsError, StateSlots

__all__ = ["OutOfPagesError", "PageAllocator", "RELEASED", "CacheManager", "CapacitySnapshot", "ReservedItem",
           "RequestCache", "StepReservation", "PrefixCache", "OutOfSlotsError", "StateSlots"]

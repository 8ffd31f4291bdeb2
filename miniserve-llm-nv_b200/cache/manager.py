"""The cache manager: who holds which pages and state slots, as plain host-side bookkeeping.

One :class:`PageAllocator` per *paged group* (layers whose mixers keep the same form of keys
and values; a group with a sliding window is separate from one that keeps everything), one
block table per request and group, one state slot per request.  A step is a transaction, as in
miniserve/kv/manager.py:119-192: :meth:`prepare` reserves the pages the step's new tokens need
and computes their slots, :meth:`commit` makes the new lengths and pages permanent (and gives
back pages that a window has passed), :meth:`abort` returns the reserved pages and leaves every
length as it was.  :meth:`release` gives back everything a request holds.

Whole pages of a prompt can be shared between requests (:mod:`.prefix`); this is on only when
every group keeps all keys and the model has no per-request state, because only then does a
page depend on nothing but the tokens before it.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy
from typing import Optional, Sequence

from ..parts.base import PagedKVNeed, StateNeed
from .allocator import OutOfPagesError, PageAllocator
from .prefix import PrefixCache, PrefixEntry
from .state_slots import StateSlots

RELEASED = -1   # block-table entry of a page that a sliding window has passed


@dataclass
class RequestCache:
    request_id: str
    slot: int
    length: int = 0
    tables: list[list[int]] = field(default_factory=list)   # per paged group: page per page index, or RELEASED


@dataclass
class ReservedItem:
    request_id: str
    start: int
    end: int
    new_pages: list[list[int]]      # per paged group
    tables: list[list[int]]         # per paged group: the table this step runs with (old + new pages)
    slots: list                     # per paged group: page * page_size + offset of every new token (a numpy array)


@dataclass
class StepReservation:
    step_id: int
    items: list[ReservedItem]
    closed: bool = False


@dataclass(frozen=True)
class CapacitySnapshot:
    """What the scheduler plans against: per paged group the pages that are free or could be freed by evicting
    reusable prefixes, and the free state slots.  The page arithmetic is here, with the cache, so that a group
    with other needs changes this class and not the scheduler; a model without paged groups fits any plan."""

    page_size: int
    total_pages: tuple[int, ...]
    free_pages: tuple[int, ...]
    reclaimable_pages: tuple[int, ...]
    free_slots: int

    def available(self) -> list[int]:
        """Per paged group: pages a step could get (free now, or held by the prefix cache alone)."""
        return [free + reclaimable for free, reclaimable in zip(self.free_pages, self.reclaimable_pages)]

    def pages_for(self, start: int, end: int) -> tuple[int, ...]:
        """Per paged group: new pages a request of ``start`` committed tokens needs to reach ``end``.  (A group
        with a window needs them as well while the step runs; what the window has passed comes back at commit.)"""
        ps = self.page_size
        need = (end + ps - 1) // ps - (start + ps - 1) // ps
        return tuple(need for _ in self.free_pages)

    def room(self, start: int, available: Sequence[int]) -> int:
        """The most tokens a request of ``start`` committed tokens can add with ``available`` pages per group."""
        ps = self.page_size
        held = (start + ps - 1) // ps
        return min(((pages + held) * ps - start for pages in available), default=1 << 60)


class CacheManager:
    def __init__(self, groups: Sequence, page_size: int, num_pages: int, max_seqs: int,
                 enable_prefix_cache: bool = False, prefix_cache_max_entries: int = 64,
                 prefix_namespace: str = "") -> None:
        if page_size < 1:
            raise ValueError("page size must be at least 1")
        self.page_size = page_size
        self.num_pages = num_pages
        self.paged_needs: list[PagedKVNeed] = [g.need for g in groups if isinstance(g.need, PagedKVNeed)]
        self.state_needs: list[StateNeed] = [g.need for g in groups if isinstance(g.need, StateNeed)]
        # position of every model group among the paged / state groups
        self.group_index: list[tuple[str, int]] = []
        paged = state = 0
        for g in groups:
            if isinstance(g.need, PagedKVNeed):
                self.group_index.append(("paged", paged))
                paged += 1
            else:
                self.group_index.append(("state", state))
                state += 1
        self.allocators = [PageAllocator(num_pages) for _ in self.paged_needs]
        self.slots = StateSlots(max_seqs)
        self.requests: dict[str, RequestCache] = {}
        self._next_step = 0
        self._open: Optional[StepReservation] = None
        shareable = all(need.window is None for need in self.paged_needs) and not self.state_needs and self.paged_needs
        self.prefix: Optional[PrefixCache] = (
            PrefixCache(prefix_namespace, page_size, prefix_cache_max_entries)
            if enable_prefix_cache and shareable else None)

    # ------------------------------------------------------------------ requests
    def admit(self, request_id: str) -> RequestCache:
        """Gives the request a state slot and empty block tables."""
        if request_id in self.requests:
            raise RuntimeError(f"request {request_id!r} is already admitted")
        slot = self.slots.allocate(request_id)
        entry = RequestCache(request_id, slot, 0, [[] for _ in self.paged_needs])
        self.requests[request_id] = entry
        return entry

    def attach_prefix(self, request_id: str, prompt: Sequence[int]) -> int:
        """Attaches cached pages that hold the start of ``prompt``; returns the tokens covered.

        At least one token of the prompt is always left to compute
        (miniserve/kv/prefix_cache.py:93-96).
        """
        entry = self.requests[request_id]
        if self.prefix is None or entry.length != 0 or any(entry.tables):
            return 0
        hits = self.prefix.lookup(prompt)
        if hits and len(hits) * self.page_size >= len(prompt):
            hits = hits[:-1]
        for hit in hits:
            for group, page in enumerate(hit.pages):
                self.allocators[group].retain(page)
                entry.tables[group].append(page)
        entry.length = len(hits) * self.page_size
        return entry.length

    def cache_prefix(self, request_id: str, prompt: Sequence[int]) -> int:
        """Offers the full pages of a completed prompt for reuse; returns how many were added."""
        entry = self.requests[request_id]
        if self.prefix is None or entry.length < len(prompt):
            return 0
        full = len(prompt) // self.page_size
        pages = [[entry.tables[g][index] for g in range(len(self.paged_needs))] for index in range(full)]
        added, replaced = self.prefix.insert(prompt, pages, self._held_by_cache_only)
        for new in added:
            for group, page in enumerate(new.pages):
                self.allocators[group].retain(page)
        for old in replaced:
            for group, page in enumerate(old.pages):
                self.allocators[group].release(page)
        return len(added)

    def release(self, request_id: str) -> None:
        """Gives back every page and the state slot of the request."""
        if self._open is not None and any(item.request_id == request_id for item in self._open.items):
            raise RuntimeError(f"request {request_id!r} is part of the open step; commit or abort first")
        entry = self.requests.pop(request_id)
        for group, table in enumerate(entry.tables):
            for page in table:
                if page != RELEASED:
                    self.allocators[group].release(page)
        self.slots.release(entry.slot)

    def length(self, request_id: str) -> int:
        return self.requests[request_id].length

    def truncate(self, request_id: str, length: int) -> None:
        """Forgets the request's tokens from position ``length`` on and gives back the pages that held only them
        (a request that drops tokens it computed ahead, or a benchmark that decodes the same steps again).  Not
        for groups with a sliding window: the pages it would have to bring back are gone."""
        if self._open is not None and any(item.request_id == request_id for item in self._open.items):
            raise RuntimeError(f"request {request_id!r} is part of the open step; commit or abort first")
        entry = self.requests[request_id]
        if not 0 <= length <= entry.length:
            raise ValueError(f"request {request_id!r} holds {entry.length} tokens; cannot truncate to {length}")
        if any(need.window is not None for need in self.paged_needs) or self.state_needs:
            raise RuntimeError("truncate needs every token's keys and no per-request state")
        keep = (length + self.page_size - 1) // self.page_size
        if length % self.page_size:
            # the request will write its next tokens into the page that holds token `length`: nobody else may hold it
            for group, table in enumerate(entry.tables):
                if self.allocators[group].refcount(table[keep - 1]) > 1:
                    raise RuntimeError(f"request {request_id!r} shares the page that holds token {length} (a reused "
                                       "prefix); truncate to a multiple of the page size instead")
        for group, table in enumerate(entry.tables):
            for page in table[keep:]:
                self.allocators[group].release(page)
            del table[keep:]
        entry.length = length

    # ------------------------------------------------------------------ capacity
    def pages_for(self, start: int, end: int) -> int:
        """New pages a request of committed length ``start`` needs to reach ``end`` (per group)."""
        ps = self.page_size
        return (end + ps - 1) // ps - (start + ps - 1) // ps

    def _held_by_cache_only(self, entry: PrefixEntry) -> bool:
        return all(self.allocators[g].refcount(p) == 1 for g, p in enumerate(entry.pages))

    def _reclaimable_entries(self) -> list[PrefixEntry]:
        """Cached pages that evicting leaves first can free: held by the cache only, and so is every entry
        behind them in their chains.  (An entry that only the cache holds can stand before one that a request
        holds: the request computed a copy of the earlier pages itself, then cached its later ones behind
        entries that were there already.)"""
        if self.prefix is None:
            return []
        entries = self.prefix.entries
        blocked: set[bytes] = set()
        for entry in entries.values():
            if self._held_by_cache_only(entry):
                continue
            digest: Optional[bytes] = entry.digest
            while digest is not None and digest in entries and digest not in blocked:
                blocked.add(digest)
                digest = entries[digest].parent
        return [e for e in entries.values() if e.digest not in blocked]

    def evictable_now(self) -> int:
        """How many cached pages :meth:`prepare` could free by evicting leaves first (what ``capacity`` reports
        as reclaimable, counted the slow way: by doing it on a copy)."""
        if self.prefix is None:
            return 0
        children = {digest: entry.children for digest, entry in self.prefix.entries.items()}
        alive = dict(self.prefix.entries)
        count = 0
        while True:
            leaf = next((e for d, e in alive.items() if children[d] == 0 and self._held_by_cache_only(e)), None)
            if leaf is None:
                return count
            del alive[leaf.digest]
            if leaf.parent in children:
                children[leaf.parent] -= 1
            count += 1

    def capacity(self) -> CapacitySnapshot:
        reclaimable = len(self._reclaimable_entries())
        return CapacitySnapshot(
            page_size=self.page_size,
            total_pages=tuple(a.num_pages for a in self.allocators),
            free_pages=tuple(a.free_count for a in self.allocators),
            reclaimable_pages=tuple(reclaimable for _ in self.allocators),
            free_slots=self.slots.free_count)

    def _make_room(self, wanted: Sequence[int]) -> None:
        """Evicts reusable prefixes nobody holds until every group has ``wanted`` free pages."""
        def short() -> bool:
            return any(a.free_count < w for a, w in zip(self.allocators, wanted))

        while short() and self.prefix is not None:
            victim = next((e for e in self.prefix.eviction_order() if self._held_by_cache_only(e)), None)
            if victim is None:
                break
            for group, page in enumerate(victim.pages):
                self.allocators[group].release(page)
            self.prefix.remove(victim)
        if short():
            raise OutOfPagesError(
                "OUT_OF_PAGES: requested=%s, free=%s" % (list(wanted), [a.free_count for a in self.allocators]))

    # ------------------------------------------------------------------ step transaction
    def prepare(self, items: Sequence[tuple[str, int]]) -> StepReservation:
        """Reserves pages for ``(request_id, number of new tokens)`` pairs; all or nothing."""
        if self._open is not None:
            raise RuntimeError("the previous step was neither committed nor aborted")
        seen: set[str] = set()
        wanted = [0] * len(self.allocators)
        plans = []
        for request_id, count in items:
            if request_id in seen:
                raise ValueError(f"request {request_id!r} appears twice in one step")
            seen.add(request_id)
            if count < 1:
                raise ValueError("a step brings at least one token per request")
            entry = self.requests[request_id]
            end = entry.length + count
            fresh = [(end + self.page_size - 1) // self.page_size - len(table) for table in entry.tables]
            for group, n in enumerate(fresh):
                wanted[group] += max(n, 0)
            plans.append((entry, end, fresh))
        self._make_room(wanted)

        reserved: list[ReservedItem] = []
        for entry, end, fresh in plans:
            new_pages = [self.allocators[g].allocate(max(n, 0)) for g, n in enumerate(fresh)]
            tables = [table + new for table, new in zip(entry.tables, new_pages)]
            slots = []
            positions = numpy.arange(entry.length, end, dtype=numpy.int64)
            for table in tables:
                pages = numpy.asarray(table, dtype=numpy.int64)[positions // self.page_size]
                if (pages == RELEASED).any():
                    raise RuntimeError("a new token falls into a page that was given back")
                slots.append(pages * self.page_size + positions % self.page_size)
            reserved.append(ReservedItem(entry.request_id, entry.length, end, new_pages, tables, slots))
        reservation = StepReservation(self._next_step, reserved)
        self._next_step += 1
        self._open = reservation
        return reservation

    def _close(self, reservation: StepReservation) -> None:
        if reservation.closed or self._open is not reservation:
            raise RuntimeError("this step is not the open one (already committed or aborted?)")
        reservation.closed = True
        self._open = None

    def commit(self, reservation: StepReservation) -> None:
        self._close(reservation)
        for item in reservation.items:
            entry = self.requests[item.request_id]
            entry.tables = [list(table) for table in item.tables]
            entry.length = item.end
            for group, need in enumerate(self.paged_needs):
                if need.window is None:
                    continue
                # the next query sits at position `length`; it sees keys from length - window + 1 on
                first_needed = entry.length - need.window + 1
                table = entry.tables[group]
                for index in range(len(table)):
                    if (index + 1) * self.page_size > first_needed:
                        break
                    if table[index] != RELEASED:
                        self.allocators[group].release(table[index])
                        table[index] = RELEASED

    def abort(self, reservation: StepReservation) -> None:
        self._close(reservation)
        for item in reservation.items:
            for group, pages in enumerate(item.new_pages):
                for page in pages:
                    self.allocators[group].release(page)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost or held twice: every page's holders are exactly the tables and entries that name it."""
        for group, allocator in enumerate(self.allocators):
            allocator.check_invariants()
            holders = [0] * allocator.num_pages
            for entry in self.requests.values():
                pages = [p for p in entry.tables[group] if p != RELEASED]
                if len(set(pages)) != len(pages):
                    raise AssertionError(f"request {entry.request_id!r} names a page twice")
                for page in pages:
                    holders[page] += 1
            if self.prefix is not None:
                for cached in self.prefix.entries.values():
                    holders[cached.pages[group]] += 1
            if self._open is not None:
                for item in self._open.items:
                    for page in item.new_pages[group]:
                        holders[page] += 1
            for page in range(allocator.num_pages):
                if holders[page] != allocator.refcount(page):
                    raise AssertionError(
                        f"group {group} page {page}: {holders[page]} holders but refcount {allocator.refcount(page)}")
        if self.evictable_now() != len(self._reclaimable_entries()):
            raise AssertionError("the reclaimable pages reported are not the pages that evicting leaves first frees")
        if self.prefix is not None and len(self.prefix.entries) > self.prefix.max_entries:
            raise AssertionError("the prefix cache holds more entries than its limit")
        self.slots.check_invariants()
        if sorted(e.slot for e in self.requests.values()) != sorted(
                s for s in range(self.slots.num_slots) if self.slots.owner(s) is not None):
            raise AssertionError("state slots and requests disagree")

"""Page allocator of one pool: a free set with reference counts.

Behaviour after miniserve/kv/allocator.py:23-79: ``allocate(n)`` hands out the ``n`` lowest
free page numbers or raises :class:`OutOfPagesError` without changing anything; ``retain``
adds a holder to a page in use; ``release`` drops one and frees the page at zero.  Releasing
or retaining a free page is an error, never a silent no-op.
"""

from __future__ import annotations

import heapq


class OutOfPagesError(RuntimeError):
    """Fewer free pages than requested."""


class PageAllocator:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free_heap = list(range(num_pages))
        self._refcount = [0] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free_heap)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free_heap)

    def refcount(self, page: int) -> int:
        return self._refcount[page]

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if count > len(self._free_heap):
            raise OutOfPagesError(f"OUT_OF_PAGES: requested={count}, free={len(self._free_heap)}")
        pages = [heapq.heappop(self._free_heap) for _ in range(count)]
        for page in pages:
            self._refcount[page] = 1
        return pages

    def retain(self, page: int) -> None:
        if self._refcount[page] <= 0:
            raise RuntimeError(f"page {page} is free and cannot be retained")
        self._refcount[page] += 1

    def release(self, page: int) -> bool:
        """Drops one holder; True if the page became free."""
        if self._refcount[page] <= 0:
            raise RuntimeError(f"page {page} is freed twice")
        self._refcount[page] -= 1
        if self._refcount[page] == 0:
            heapq.heappush(self._free_heap, page)
            return True
        return False

    def check_invariants(self) -> None:
        free = sorted(self._free_heap)
        if len(set(free)) != len(free):
            raise AssertionError("a page is in the free set twice")
        for page in range(self.num_pages):
            is_free = self._refcount[page] == 0
            if is_free != (page in set(free)):
                raise AssertionError(f"page {page}: refcount {self._refcount[page]} disagrees with the free set")

"""Reuse of whole pages between requests that start with the same tokens.

After miniserve/kv/prefix_cache.py:39-133: a full page of prompt tokens is named by a chained
SHA-256 over (namespace, digest of the page before it, the page's tokens); an entry keeps the
page numbers (one per layer group) and the tokens themselves, which are compared again on a
hit.  The cache holds one reference on every page it names.  Entries whose pages nobody else
holds are *reclaimable*: when a step needs pages they are evicted, least recently used first,
leaves of the chain before their parents.  The cache holds at most ``max_entries`` entries: an
insert beyond that replaces reclaimable leaves, least recently used first
(prefix_cache.py:122-125 drops the oldest entries there), and caches no further page of the
prompt once nothing can be replaced.
"""

from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence


def page_digest(namespace: bytes, previous: bytes, tokens: Sequence[int]) -> bytes:
    h = hashlib.sha256()
    h.update(struct.pack("<I", len(namespace)))
    h.update(namespace)
    h.update(previous)
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    return h.digest()


@dataclass
class PrefixEntry:
    digest: bytes
    parent: Optional[bytes]
    tokens: tuple[int, ...]
    pages: tuple[int, ...]          # one page per paged group
    last_used: int = 0
    children: int = 0


class PrefixCache:
    def __init__(self, namespace: str, page_size: int, max_entries: int) -> None:
        self.namespace = namespace.encode()
        self.page_size = page_size
        self.max_entries = max_entries
        self.entries: dict[bytes, PrefixEntry] = {}
        self._clock = 0

    def _tick(self) -> int:
        self._clock += 1
        return self._clock

    def lookup(self, tokens: Sequence[int]) -> list[PrefixEntry]:
        """Entries for the leading full pages of ``tokens`` that are cached, in order."""
        found: list[PrefixEntry] = []
        previous = b""
        for start in range(0, len(tokens) - self.page_size + 1, self.page_size):
            chunk = tuple(tokens[start:start + self.page_size])
            digest = page_digest(self.namespace, previous, chunk)
            entry = self.entries.get(digest)
            if entry is None or entry.tokens != chunk:
                break
            found.append(entry)
            previous = digest
        now = self._tick()
        for entry in found:
            entry.last_used = now
        return found

    def insert(self, tokens: Sequence[int], pages_per_page_index: Sequence[Sequence[int]],
               replaceable: Optional[Callable[[PrefixEntry], bool]] = None) -> tuple[list[PrefixEntry], list[PrefixEntry]]:
        """Adds entries for the full pages of ``tokens`` not cached yet; returns (new entries, replaced entries).

        ``pages_per_page_index[i]`` are the page numbers (one per group) that hold page ``i``.
        The caller retains the pages of every new entry and releases those of every replaced one.
        At ``max_entries`` a new entry takes the place of the least recently used leaf for which
        ``replaceable(entry)`` holds (no ``replaceable``: none is) and which is not part of the
        chain being inserted; if there is none, the rest of the prompt stays uncached.
        """
        added: list[PrefixEntry] = []
        replaced: list[PrefixEntry] = []
        previous: bytes = b""
        parent: Optional[PrefixEntry] = None
        now = self._tick()
        chain: set[bytes] = set()
        full_pages = len(tokens) // self.page_size
        for index in range(full_pages):
            chunk = tuple(tokens[index * self.page_size:(index + 1) * self.page_size])
            digest = page_digest(self.namespace, previous, chunk)
            entry = self.entries.get(digest)
            if entry is None:
                if len(self.entries) >= self.max_entries:
                    victim = None
                    if replaceable is not None:
                        victim = next((e for e in self.eviction_order()
                                       if e.digest not in chain and replaceable(e)), None)
                    if victim is None:
                        break
                    self.remove(victim)
                    replaced.append(victim)
                entry = PrefixEntry(digest, parent.digest if parent else None, chunk,
                                    tuple(pages_per_page_index[index]), now)
                self.entries[digest] = entry
                if parent is not None:
                    parent.children += 1
                added.append(entry)
            elif entry.tokens != chunk:
                break
            else:
                entry.last_used = now
            chain.add(digest)
            parent, previous = entry, digest
        return added, replaced

    def eviction_order(self) -> list[PrefixEntry]:
        """Leaves of the chains, least recently used first."""
        return sorted((e for e in self.entries.values() if e.children == 0), key=lambda e: e.last_used)

    def remove(self, entry: PrefixEntry) -> None:
        del self.entries[entry.digest]
        if entry.parent is not None and entry.parent in self.entries:
            self.entries[entry.parent].children -= 1

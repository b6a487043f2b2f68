"""Host-side bookkeeping of the cache: which pages are free, which slot holds which pages.

Nothing here touches the device; the tables built here are mirrored into device
tensors by ``cache.Cache``.  The reference gives each sequence one session with its own
key/value arrays of the full context length (src/model_session.c:260-446) and resets it by
zeroing them (src/session.c:113-172); here sequences share a pool of pages of 64 tokens, a
sequence holds only the pages its length needs, and a freed page needs no clearing because
reads are bounded by the sequence's length.
"""
from __future__ import annotations

from typing import Dict, List

PAGE = 64


class CacheError(RuntimeError):
    """Misuse of the cache: a slot or page held twice, freed twice, or unknown."""


class CacheFull(CacheError):
    """No free page or slot is left for what was asked."""


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


class PagePool:
    """Free list over ``n_pages`` page ids.  Every id is either free or held, never both."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise CacheError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise CacheFull(f"{n} pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise CacheError(f"page {p} was on the free list while held")
            self._held[p] = True
        return out

    def free(self, pages: List[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise CacheError(f"page {p} does not exist")
            if not self._held[p]:
                raise CacheError(f"page {p} is freed twice")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is exactly once either free or held."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in set(self._free)):
                raise CacheError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class SlotTable:
    """Slots for sequences: a slot is free or holds one sequence with its length."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise CacheError(f"a cache needs at least one slot, got {n_slots}")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._active: Dict[int, int] = {}  # slot -> length

    @property
    def n_free(self) -> int:
        return len(self._free)

    def active(self) -> List[int]:
        return sorted(self._active)

    def open(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} slots are in use")
        s = self._free.pop()
        if s in self._active:
            raise CacheError(f"slot {s} is handed out twice")
        self._active[s] = 0
        return s

    def close(self, slot: int) -> None:
        if slot not in self._active:
            raise CacheError(f"slot {slot} is not open (closed twice, or never opened)")
        del self._active[slot]
        self._free.append(slot)

    def length(self, slot: int) -> int:
        try:
            return self._active[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not open") from None

    def set_length(self, slot: int, n: int) -> None:
        if slot not in self._active:
            raise CacheError(f"slot {slot} is not open")
        self._active[slot] = n

    def check(self) -> None:
        if len(set(self._free)) != len(self._free):
            raise CacheError("a slot is on the free list twice")
        if set(self._free) & set(self._active):
            raise CacheError("a slot is both free and open")
        if len(self._free) + len(self._active) != self.n_slots:
            raise CacheError("a slot is lost")

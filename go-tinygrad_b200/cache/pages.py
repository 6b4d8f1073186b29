"""Host-side bookkeeping of the cache: which slots and which pages are in use.

A *slot* belongs to one sequence from the step that starts it until the batch
ends; a *page* holds 64 consecutive tokens of one sequence.  Both allocators
refuse to hand out what is taken, to take back what is free, and can say at any
time what is in use -- the properties the tests check (no slot lost, held twice
or freed twice).  Pure Python: no device is touched here.

The reference has one sequence at a time and a buffer of 2048 positions per
layer that is never given back (model/gpu_forward.go:477-496); slots and pages
are this library's.
"""
from __future__ import annotations

from typing import Dict, List


class CacheFull(RuntimeError):
    """No free slot or page is left for what was asked."""


class CacheMisuse(RuntimeError):
    """A slot or page was freed twice, or used without being held."""


class SlotTable:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("the cache needs at least one slot")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))   # pop() gives the lowest first
        self._held = [False] * n_slots

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        slot = self._free.pop()
        if self._held[slot]:
            raise CacheMisuse(f"slot {slot} was on the free list while held")
        self._held[slot] = True
        return slot

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots:
            raise CacheMisuse(f"slot {slot} does not exist")
        if not self._held[slot]:
            raise CacheMisuse(f"slot {slot} is freed but is not held")
        self._held[slot] = False
        self._free.append(slot)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._held[slot]

    @property
    def n_free(self) -> int:
        return len(self._free)

    def held(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._held[s]]


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("the cache needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._owner: Dict[int, int] = {}           # page -> slot

    def alloc(self, n: int, slot: int) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{n} more cache pages are needed but {len(self._free)} of "
                            f"{self.n_pages} are free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            if p in self._owner:
                raise CacheMisuse(f"page {p} was on the free list while owned by slot {self._owner[p]}")
            self._owner[p] = slot
        return pages

    def free(self, pages: List[int], slot: int) -> None:
        for p in pages:
            if self._owner.get(p) != slot:
                raise CacheMisuse(f"page {p} is freed by slot {slot} but belongs to "
                                  f"{self._owner.get(p, 'nobody')}")
            del self._owner[p]
            self._free.append(p)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def owned_by(self, slot: int) -> List[int]:
        return sorted(p for p, s in self._owner.items() if s == slot)

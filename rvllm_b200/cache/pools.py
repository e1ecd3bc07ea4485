"""Page pool and slot pool: plain free lists with owner bookkeeping.

The reference has the page layout only (v3/crates/rvllm-mem/src/kv_layout.rs:10-47) and
static identity block tables (v3/crates/rvllm-runtime/src/bring_up.rs:420-435); its scheduler
spec names an allocator (v3/specs/07-scheduler.md:76,97) that was never written.  The free
list is a stack, so a page given back is the next one handed out.
"""
from __future__ import annotations

from typing import Hashable, List, Optional

from ..errors import KvExhausted, SchedulerError


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise SchedulerError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # page 0 on top
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int, owner: Hashable) -> List[int]:
        if n > len(self._free):
            raise KvExhausted(n, len(self._free))
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            if self._owner[p] is not None:
                raise SchedulerError(f"page {p} was on the free list while held by {self._owner[p]!r}")
            self._owner[p] = owner
        return pages

    def release(self, pages, owner: Hashable) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise SchedulerError(f"page {p} does not exist")
            if self._owner[p] is None:
                raise SchedulerError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise SchedulerError(f"page {p} is held by {self._owner[p]!r}, not by {owner!r}")
            self._owner[p] = None
            self._free.append(p)

    def owner(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free once or held once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise SchedulerError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise SchedulerError(f"page {p} is {'both free and held' if p in free else 'lost'}")


class SlotPool:
    """Slots of fixed-size per-request state."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._owner: List[Optional[Hashable]] = [None] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, owner: Hashable) -> int:
        if not self._free:
            raise SchedulerError(f"all {self.num_slots} request slots are taken")
        s = self._free.pop()
        self._owner[s] = owner
        return s

    def release(self, slot: int, owner: Hashable) -> None:
        if self._owner[slot] != owner or self._owner[slot] is None:
            raise SchedulerError(f"slot {slot} is not held by {owner!r}")
        self._owner[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise SchedulerError("a slot is on the free list twice")
        for s in range(self.num_slots):
            if (s in free) == (self._owner[s] is not None):
                raise SchedulerError(f"slot {s} is {'both free and held' if s in free else 'lost'}")

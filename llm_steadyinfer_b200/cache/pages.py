"""Page pool: the free list and reference counts of one group's pages.

Modelled on the reference's ``BlockAllocator`` (src/source/scheduler/block_allocator.cpp:
LIFO free list handing out ascending ids first :15-19, per-block reference counts,
all-or-nothing allocation :44-75, release when the count reaches zero :98-111), without its
fixed-width table rows: tables are per request and live in the cache manager.

A page whose count reaches zero while it carries a content hash (prefix reuse) is parked in
a second free list and loses its hash only when it is handed out again, oldest first.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, List, Optional


class PageError(RuntimeError):
    """A page was released twice, retained while free, or is outside the pool."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() -> 0, 1, 2, ...
        self._parked: "OrderedDict[int, None]" = OrderedDict()            # free but still hashed
        self._ref = [0] * self.num_pages
        self.on_evict: Optional[Callable[[int], None]] = None            # parked page is reused

    @property
    def num_free(self) -> int:
        return len(self._free) + len(self._parked)

    def refcount(self, page: int) -> int:
        return self._ref[page]

    def allocate(self, n: int) -> Optional[List[int]]:
        """n pages with count 1 each, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > self.num_free:
            return None
        out = []
        for _ in range(n):
            if self._free:
                p = self._free.pop()
            else:
                p, _ = self._parked.popitem(last=False)
                if self.on_evict:
                    self.on_evict(p)
            self._ref[p] = 1
            out.append(p)
        return out

    def retain(self, page: int) -> None:
        """One more holder of a page: a live one, or a parked one that is taken back."""
        self._check(page)
        if self._ref[page] == 0:
            if page not in self._parked:
                raise PageError(f"page {page} is free and carries no content; it cannot be retained")
            del self._parked[page]
        self._ref[page] += 1

    def release(self, page: int, park: bool = False) -> None:
        self._check(page)
        if self._ref[page] <= 0:
            raise PageError(f"page {page} released while already free")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            if park:
                self._parked[page] = None
            else:
                self._free.append(page)

    def is_parked(self, page: int) -> bool:
        return page in self._parked

    def _check(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise PageError(f"page {page} is outside the pool of {self.num_pages}")

    def check_invariant(self, held: List[int]) -> None:
        """``held`` lists every page reference that tables hold (a shared page once per
        holder). Raises unless each page is either free exactly once or held exactly
        refcount times."""
        counts = [0] * self.num_pages
        for p in held:
            self._check(p)
            counts[p] += 1
        free_seen = [0] * self.num_pages
        for p in list(self._free) + list(self._parked):
            free_seen[p] += 1
        for p in range(self.num_pages):
            if counts[p] != self._ref[p]:
                raise PageError(f"page {p}: held {counts[p]} times but its count is {self._ref[p]}")
            if self._ref[p] == 0 and free_seen[p] != 1:
                raise PageError(f"page {p}: unheld but on the free lists {free_seen[p]} times (lost or doubled)")
            if self._ref[p] > 0 and free_seen[p] != 0:
                raise PageError(f"page {p}: held and free at once")


class SlotPool:
    """Slots for per-request state of fixed size; a request keeps one from admission to its end."""

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._used = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._used.add(s)
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._used:
            raise PageError(f"state slot {slot} given back while not in use")
        self._used.remove(slot)
        self._free.append(slot)

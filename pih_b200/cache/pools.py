"""Page pool and state-slot pool: who holds what, checked on every call.

The reference's pool (plugins/model-qwen3/qwen3_kv_slot_pool.cpp:67-364) walks
each 16-token page through seven lifecycle states with a zeroing pass before
reuse and hands out generation-stamped handles.  Here a page is either free
or held by exactly one owner; reuse needs no zeroing because attention never
reads beyond a request's length.  Every call checks the invariants that the
reference's states guard: no page is handed out twice, freed twice, or freed
by someone who does not hold it; an allocation that cannot be met changes
nothing (qwen3_kv_slot_pool_test.cpp:69 "exhaustion leaves state untouched").
"""
from __future__ import annotations

from typing import Hashable, List


class OutOfPages(RuntimeError):
    """The pool cannot supply the pages asked for; nothing was allocated."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        # most recently freed page is reused first: reuse shows up early in tests
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._owner: List[Hashable] = [None] * num_pages
        self.pages_handed_out = 0          # over the pool's life; exceeds num_pages once pages are reused

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, count: int, owner: Hashable) -> List[int]:
        if owner is None:
            raise ValueError("pages need an owner")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            if self._owner[p] is not None:
                raise AssertionError(f"page {p} was free and owned by {self._owner[p]!r} at once")
            self._owner[p] = owner
        self.pages_handed_out += count
        return pages

    def free(self, pages, owner: Hashable) -> None:
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not in the pool")
            if self._owner[p] is None:
                raise ValueError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise ValueError(f"page {p} belongs to {self._owner[p]!r}, not to {owner!r}")
        if len(set(pages)) != len(pages):
            raise ValueError("a page is named twice in one free")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """No page lost, none both free and held."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise AssertionError(f"page {p}: free={p in free}, owner={self._owner[p]!r}")


class OutOfSlots(RuntimeError):
    pass


class StateSlotPool:
    """Slots for per-request state of fixed size (one slot per live request)."""

    def __init__(self, num_slots: int):
        if num_slots < 1:
            raise ValueError("a slot pool needs at least one slot")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._owner: List[Hashable] = [None] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, owner: Hashable) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} state slots are taken")
        s = self._free.pop()
        self._owner[s] = owner
        return s

    def release(self, slot: int, owner: Hashable) -> None:
        if not 0 <= slot < self.num_slots or self._owner[slot] is None:
            raise ValueError(f"state slot {slot} is released twice or was never taken")
        if self._owner[slot] != owner:
            raise ValueError(f"state slot {slot} belongs to {self._owner[slot]!r}, not to {owner!r}")
        self._owner[slot] = None
        self._free.append(slot)

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a slot is on the free list twice")
        for s in range(self.num_slots):
            if (s in free) == (self._owner[s] is not None):
                raise AssertionError(f"slot {s}: free={s in free}, owner={self._owner[s]!r}")

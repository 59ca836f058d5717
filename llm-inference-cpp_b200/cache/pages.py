"""Host-side bookkeeping of the cache: slots, pages, lengths.

The reference keeps one ``KVCache`` object per sequence with a fixed capacity
(include/llmi/model/transformer.hpp:29-45; src/model/transformer.cpp:182-190).
Here many sequences share one pool: a *slot* stands for one live sequence, and
its keys and values lie in *pages* of ``page_size`` positions taken from the pool
as the sequence grows and given back when its slot is freed.  The errors keep the
reference's meaning ("cache is full", src/model/transformer.cpp:208).

This file is pure bookkeeping (no tensors): it can be tested without a GPU.
"""
from __future__ import annotations

PAGE_SIZE = 64


class CacheError(RuntimeError):
    pass


def pages_for(tokens: int, page_size: int = PAGE_SIZE) -> int:
    return (tokens + page_size - 1) // page_size


class SlotTable:
    """Which slots are live.  A slot is handed out once until it is freed."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise CacheError("cache: needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))   # pop() hands out the lowest free slot
        self._live = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheError("cache is full: no free slot")
        s = self._free.pop()
        self._live.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._live:
            raise CacheError(f"cache: slot {slot} is not live (freed twice or never allocated)")
        self._live.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    def all_live(self, slots) -> bool:
        return self._live.issuperset(slots)

    @property
    def live(self) -> set:
        return set(self._live)

    @property
    def n_free(self) -> int:
        return len(self._free)


class PagePool:
    """Pages of one cache group: a free list and, per slot, the pages it holds in position order.

    ``window`` > 0 means a query only needs the last ``window`` positions: pages that lie
    wholly before the window of the next token are given back early and their table entries
    become -1.
    """

    def __init__(self, n_pages: int, page_size: int = PAGE_SIZE, window: int = 0, n_slots: int = 0,
                 max_pages_per_slot: int = 0):
        if n_pages <= 0:
            raise CacheError("cache: needs at least one page")
        self.n_pages = n_pages
        self.page_size = page_size
        self.window = window
        self._free = list(range(n_pages - 1, -1, -1))
        self._pages: dict[int, list[int]] = {}     # slot -> page ids by position (-1: released)
        self._length: dict[int, int] = {}
        self._released: dict[int, int] = {}        # slot -> how many leading pages of its table were given back
        # the same tables as one int32 matrix [slot, page], kept in step with the lists, so that a step can
        # gather the page tables of its sequences with one indexing operation
        self.matrix = None
        if n_slots > 0 and max_pages_per_slot > 0:
            import numpy as np
            self.matrix = np.full((n_slots, max_pages_per_slot), -1, dtype=np.int32)

    # -- slots -----------------------------------------------------------------------------
    def open(self, slot: int) -> None:
        if slot in self._pages:
            raise CacheError(f"cache: slot {slot} is already open in this group")
        self._pages[slot] = []
        self._length[slot] = 0
        self._released[slot] = 0
        if self.matrix is not None and slot < self.matrix.shape[0]:
            self.matrix[slot, :] = -1

    def close(self, slot: int) -> None:
        if slot not in self._pages:
            raise CacheError(f"cache: slot {slot} is not open in this group")
        for p in self._pages.pop(slot):
            if p >= 0:
                self._free.append(p)
        del self._length[slot]
        del self._released[slot]
        if self.matrix is not None and slot < self.matrix.shape[0]:
            self.matrix[slot, :] = -1

    # -- growth ----------------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> int:
        have = len(self._pages[slot])
        return max(0, pages_for(self._length[slot] + n_new, self.page_size) - have)

    def releasable(self, slot: int) -> int:
        """Pages of a slot that lie wholly before the window of its NEXT position: what its next growth gives
        back before it takes anything (0 without a window)."""
        if self.window <= 0:
            return 0
        first_needed = self._length[slot] - self.window + 1
        dead = min(len(self._pages[slot]), max(0, first_needed) // self.page_size)
        return max(0, dead - self._released[slot])

    def release_dead(self, slot: int) -> int:
        """Give back what :meth:`releasable` counts; returns how many pages that were."""
        n = self.releasable(slot)
        if n:
            self._release_before(slot, self._length[slot] - self.window + 1)
        return n

    def page_events(self, bases, slots=None):
        """For sequences of lengths ``bases`` (an integer array) that grow by one position: which of them
        take a new page, and how many pages each gives back first (a window's oldest pages out of reach; with
        ``slots`` the exact count for these slots — after a long prompt that can be several at once —, without
        them the one page that falls out when the window's start crosses a page end)."""
        import numpy as np
        takes = (bases % self.page_size) == 0
        if self.window <= 0:
            gives = np.zeros(len(bases), dtype=np.int64)
        elif slots is not None:
            gives = np.fromiter((self.releasable(s) for s in slots), dtype=np.int64, count=len(bases))
        else:
            first_needed = bases - self.window + 1
            gives = ((first_needed > 0) & ((first_needed % self.page_size) == 0)).astype(np.int64)
        return takes, gives

    def grow_quietly(self, slot: int) -> None:
        """One more position for a slot whose growth neither takes nor gives a page."""
        self._length[slot] += 1

    def extend(self, slot: int, n_new: int) -> int:
        """Make room for ``n_new`` more positions; returns the position of the first of them."""
        if slot not in self._pages:
            raise CacheError(f"cache: slot {slot} is not open in this group")
        base = self._length[slot]
        need = self.pages_needed(slot, n_new)
        if need > len(self._free) + self.releasable(slot):
            raise CacheError("cache is full")          # nothing has changed
        self.release_dead(slot)
        for _ in range(need):
            page = self._free.pop()
            if self.matrix is not None and slot < self.matrix.shape[0] and len(self._pages[slot]) < self.matrix.shape[1]:
                self.matrix[slot, len(self._pages[slot])] = page
            self._pages[slot].append(page)
        self._length[slot] = base + n_new
        return base

    def shrink_by_one(self, slot: int) -> None:
        """Take back the newest position of a slot (the undo of ``extend(slot, 1)``; pools without a window only:
        a window's growth may have given pages back, which cannot be undone)."""
        if self.window > 0:
            raise CacheError("cache: a windowed group cannot take a position back")
        n = self._length[slot] - 1
        if n < 0:
            raise CacheError(f"cache: slot {slot} holds no position to take back")
        if n % self.page_size == 0:            # the position opened a page: the page goes back to where it came from
            page = self._pages[slot].pop()
            self._free.append(page)
            i = len(self._pages[slot])
            if self.matrix is not None and slot < self.matrix.shape[0] and i < self.matrix.shape[1]:
                self.matrix[slot, i] = -1
        self._length[slot] = n

    def _release_before(self, slot: int, first_needed: int) -> None:
        table = self._pages[slot]
        for i in range(min(len(table), max(0, first_needed) // self.page_size)):
            if table[i] >= 0:
                self._free.append(table[i])
                table[i] = -1
                self._released[slot] = max(self._released[slot], i + 1)
                if self.matrix is not None and slot < self.matrix.shape[0] and i < self.matrix.shape[1]:
                    self.matrix[slot, i] = -1

    # -- views -----------------------------------------------------------------------------
    def length(self, slot: int) -> int:
        return self._length[slot]

    def table(self, slot: int) -> list[int]:
        return self._pages[slot]

    @property
    def n_free(self) -> int:
        return len(self._free)

    def check(self) -> None:
        """Every page is free or held by exactly one slot; none is lost."""
        seen = list(self._free)
        for table in self._pages.values():
            seen.extend(p for p in table if p >= 0)
        if sorted(seen) != list(range(self.n_pages)):
            lost = set(range(self.n_pages)) - set(seen)
            dup = {p for p in seen if seen.count(p) > 1}
            raise CacheError(f"cache: page accounting broken (lost {sorted(lost)}, held twice {sorted(dup)})")

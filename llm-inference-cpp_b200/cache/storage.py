"""Device storage of the cache and the object a step function works with.

A mixer says what it needs per sequence with a *request*:

* :class:`KVRequest` — keys and values of every position (or of a window of them),
  ``n_kv_heads × head_dim`` each.  Calls with equal requests share a *group*: one
  page pool and one pair of tensors ``[calls, pages, kv_heads, page_size, head_dim]``
  (one (page, kv head) tile is contiguous — head-major within the page, after the
  reference's layout, include/llmi/model/transformer.hpp:39-44).
* :class:`StateRequest` — a fixed-size state per sequence, ``[calls, slots, *shape]``,
  zeroed when a slot is handed out.  The Llama architecture asks for none; the slab is
  here so that a mixer with a recurrent state needs no change of the cache.

Groups with different requests have storage and page pools of their own.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import numpy as np
import torch

from .pages import PAGE_SIZE, CacheError, PagePool, SlotTable, pages_for


@dataclass(frozen=True)
class KVRequest:
    n_kv_heads: int
    head_dim: int
    window: int = 0          # 0: all positions


@dataclass(frozen=True)
class StateRequest:
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class CacheBinding:
    """What one scheduled call holds of the cache: its group and its index inside the group."""
    group: object
    index: int
    writes: bool = True      # False: the call reads another call's entries


class KVGroup:
    def __init__(self, request: KVRequest, n_calls: int, n_pages: int, page_size: int, dtype, device, n_slots: int = 0,
                 max_pages_per_slot: int = 0):
        self.request = request
        self.n_calls = n_calls
        self.page_size = page_size
        self.pool = PagePool(n_pages, page_size, request.window, n_slots, max_pages_per_slot)
        shape = (n_calls, n_pages, request.n_kv_heads, page_size, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def bytes_per_token(self) -> int:
        r = self.request
        return 2 * self.n_calls * r.n_kv_heads * r.head_dim * self.k.element_size()


class StateGroup:
    def __init__(self, request: StateRequest, n_calls: int, n_slots: int, device):
        self.request = request
        self.n_calls = n_calls
        self.data = torch.zeros((n_calls, n_slots, *request.shape), dtype=request.dtype, device=device)

    def reset(self, slot: int) -> None:
        self.data[:, slot].zero_()


_cache_serials = itertools.count(1)


class SequenceCache:
    """Slots, their lengths, and the groups' storage.  Sized by the most tokens held at once.

    ``serial`` numbers the caches of a process: unlike ``id(cache)`` it is never handed out again, so
    whatever remembers device addresses of a cache (a recorded graph) can tell it from a later one."""

    def __init__(self, kv_requests, state_requests, max_tokens: int, max_positions: int, dtype, device,
                 page_size: int = PAGE_SIZE, n_slots: int | None = None):
        """``kv_requests`` / ``state_requests``: lists of (request, number of calls)."""
        if max_tokens < page_size:
            raise CacheError(f"cache: max_tokens must be at least one page ({page_size} tokens)")
        self.serial = next(_cache_serials)
        self.page_size = page_size
        self.max_positions = max_positions
        n_pages = max_tokens // page_size
        self.n_slots = n_slots if n_slots is not None else n_pages
        self.slots = SlotTable(self.n_slots)
        self.max_pages_per_seq = min(pages_for(max_positions, page_size), n_pages)
        self.kv_groups = [KVGroup(r, n, n_pages, page_size, dtype, device, self.n_slots, self.max_pages_per_seq)
                          for r, n in kv_requests]
        self.state_groups = [StateGroup(r, n, self.n_slots, device) for r, n in state_requests]
        self._length: dict[int, int] = {}
        self._ahead: tuple = ()          # slots whose next position is reserved already (see speculate_each_by_one)
        self.device = device
        self.dtype = dtype

    # -- slots -----------------------------------------------------------------------------
    def alloc_slot(self) -> int:
        self.settle()
        slot = self.slots.alloc()
        for g in self.kv_groups:
            g.pool.open(slot)
        for g in self.state_groups:
            g.reset(slot)
        self._length[slot] = 0
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)          # raises on a slot that is not live
        if slot in self._ahead:        # everything the slot holds goes back below, a reserved next position included
            self._ahead = tuple(s for s in self._ahead if s != slot)
        for g in self.kv_groups:
            g.pool.close(slot)
        del self._length[slot]

    def length(self, slot: int) -> int:
        """Positions the slot holds (a position reserved ahead of its step does not count)."""
        if slot not in self._length:
            raise CacheError(f"cache: slot {slot} is not live")
        return self._length[slot] - (1 if slot in self._ahead else 0)

    # -- one step ahead --------------------------------------------------------------------
    # While the device runs a decode step, the host can already lay out the next one — positions, lengths, page
    # tables — if the same sequences go on; only their tokens are missing.  That needs the next positions reserved
    # before it is known whether the step will come.  The reservation is invisible (``length`` does not count it) and
    # is taken back (``settle``) by whatever touches the cache next, unless the expected step arrives and commits it.
    def can_speculate(self) -> bool:
        return all(g.pool.window == 0 for g in self.kv_groups)

    def speculate_each_by_one(self, slots) -> "np.ndarray":
        """Reserve one more position for every slot of ``slots`` ahead of its step; returns the positions.
        Raises (and reserves nothing) where :meth:`extend_each_by_one` would."""
        self.settle()
        if not self.can_speculate():
            raise CacheError("cache: a windowed group cannot reserve ahead")
        bases = self._extend_each_by_one(slots)
        self._ahead = tuple(slots)
        return bases

    def commit_speculation(self) -> None:
        """The step the positions were reserved for has come: they count from now on."""
        self._ahead = ()

    def settle(self) -> None:
        """Take back positions that were reserved ahead of a step that has not come."""
        if self._ahead:
            ahead, self._ahead = self._ahead, ()
            for s in ahead:
                if s in self._length:
                    for g in self.kv_groups:
                        g.pool.shrink_by_one(s)
                    self._length[s] -= 1

    # -- growth ----------------------------------------------------------------------------
    def can_extend(self, wanted: dict) -> None:
        """Raise unless every slot of ``wanted`` (slot → new tokens) fits, in every group.  A windowed group
        counts the pages its slots give back before they take new ones."""
        self.settle()
        for slot, n_new in wanted.items():
            if slot not in self._length:
                raise CacheError(f"cache: slot {slot} is not live")
            if self._length[slot] + n_new > self.max_positions:
                raise CacheError("sequence longer than the model's context")
        for g in self.kv_groups:
            need = sum(g.pool.pages_needed(s, n) for s, n in wanted.items())
            if need > g.pool.n_free + sum(g.pool.releasable(s) for s in wanted):
                raise CacheError("cache is full")

    def extend(self, slot: int, n_new: int) -> int:
        """Reserve room for ``n_new`` positions of a slot; returns its first new position."""
        self.can_extend({slot: n_new})
        base = self._length[slot]
        for g in self.kv_groups:
            g.pool.extend(slot, n_new)
        self._length[slot] = base + n_new
        return base

    def extend_all(self, wanted: dict) -> list:
        """Reserve room for a whole step (slot → new tokens) or, if it does not fit, raise with NOTHING changed:
        the check covers every slot and every group first; then every group first takes back the pages its
        slots no longer need and only then hands out new ones, so that no slot finds the pool empty because a
        later slot has not given its pages back yet.  Returns the first new position of each slot."""
        self.can_extend(wanted)
        for g in self.kv_groups:
            if g.pool.window > 0:
                for s in wanted:
                    g.pool.release_dead(s)
            for s, n in wanted.items():
                g.pool.extend(s, n)
        bases = []
        for s, n in wanted.items():
            bases.append(self._length[s])
            self._length[s] += n
        return bases

    def extend_each_by_one(self, slots) -> "np.ndarray":
        """One more position for every slot of ``slots`` (distinct, live): the decode step's growth, with the
        checks of :meth:`can_extend` and without a loop over the slots that need no page.  Nothing changes
        if it raises.  Returns the new positions."""
        self.settle()
        return self._extend_each_by_one(slots)

    def _extend_each_by_one(self, slots) -> "np.ndarray":
        if not self.slots.all_live(slots):
            bad = next(s for s in slots if not self.slots.is_live(s))
            raise CacheError(f"cache: slot {bad} is not live")
        length = self._length
        bases = np.fromiter((length[s] for s in slots), dtype=np.int64, count=len(slots))
        if int(bases.max()) + 1 > self.max_positions:
            raise CacheError("sequence longer than the model's context")
        events = []
        for g in self.kv_groups:
            takes, gives = g.pool.page_events(bases, slots)
            if int(takes.sum()) > g.pool.n_free + int(gives.sum()):
                raise CacheError("cache is full")
            events.append((takes, gives))
        for g, (takes, gives) in zip(self.kv_groups, events):
            pool = g.pool
            if gives.any():
                for s, n in zip(slots, gives):
                    if n:
                        pool.release_dead(s)
            if takes.any():
                for s, e in zip(slots, takes):
                    if e:
                        pool.extend(s, 1)
                    else:
                        pool.grow_quietly(s)
            else:
                for s in slots:
                    pool.grow_quietly(s)
        for s in slots:
            length[s] += 1
        return bases

    # -- accounting ------------------------------------------------------------------------
    def check(self) -> None:
        for g in self.kv_groups:
            g.pool.check()

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.kv_groups)

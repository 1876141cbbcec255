"""Paged key/value bookkeeping: page pools per layer group, block tables per request.

The reference gives every sequence one contiguous K and V buffer of the whole
context (src/model.c:3089-3101) and never frees per request; "which rows are
valid" is the sequence's position (src/engine.h:40).  Here a request holds
fixed-size pages instead.  Layers are collected in *groups* by what they keep:
all keys (``window is None``) or the last ``window`` keys (the reference's
per-layer sliding flag, src/model.h:229-235).  Every group has a pool of its
own and every request a block table per group.  Pages go back to the pool
when a request ends, and -- in a window group -- as soon as every position in
the page lies behind the window of every query still to come.

This module is host bookkeeping only (no tensors of keys or values): the
device arrays are owned by ``cache.storage``.  Nothing here is zeroed on
reuse; validity is the request's length.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np


class OutOfPages(RuntimeError):
    """A reservation did not fit; nothing was taken."""


class CacheError(RuntimeError):
    """A call that breaks the manager's rules (double free, unknown request...)."""


@dataclass(frozen=True)
class GroupSpec:
    """Layers with the same need.  `window` None keeps every key."""
    name: str
    window: Optional[int] = None


class PagePool:
    """A stack of free page numbers with a record of who holds what."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError("a pool needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held = np.zeros(n_pages, dtype=bool)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("pool is empty")
        p = self._free.pop()
        self._held[p] = True
        return p

    def give(self, page: int) -> None:
        if page < 0 or page >= self.n_pages or not self._held[page]:
            raise CacheError(f"page {page} is given back but not held")
        self._held[page] = False
        self._free.append(page)


class _Request:
    __slots__ = ("slot", "length", "reserved", "first_live_page")

    def __init__(self, slot: int, n_groups: int):
        self.slot = slot
        self.length = 0            # tokens whose keys are in the cache
        self.reserved = 0          # tokens reserved beyond `length` for the step in flight
        self.first_live_page = [0] * n_groups   # per group: table entries below this were released


class CacheManager:
    """Pages, block tables and state slots of all live requests.

    Life of a request: ``open`` (takes a state slot) -> any number of
    ``reserve(n)`` / ``commit`` pairs (a step that was planned but did not run
    is undone with ``cancel``) -> ``close``.  ``reserve`` is atomic over all
    groups: it takes every page the next `n` tokens need, or none.
    """

    def __init__(self, groups: Sequence[GroupSpec], n_pages: int, page_size: int,
                 max_requests: int, max_request_tokens: int):
        if page_size < 1:
            raise CacheError("page_size must be >= 1")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_pages_per_request = -(-max_request_tokens // page_size)
        self.pools = [PagePool(n_pages) for _ in self.groups]
        # block tables: [group][slot, page index] -> page number, -1 where none is held
        self.tables = [np.full((max_requests, self.max_pages_per_request), -1, dtype=np.int32)
                       for _ in self.groups]
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[object, _Request] = {}
        self.generation = np.zeros(max_requests, dtype=np.int64)   # bumped when a slot is assigned
        self.high_water = [0] * len(self.groups)

    # ---- requests and slots ------------------------------------------------
    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def open(self, request_id) -> int:
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise OutOfPages("no free request slot")
        slot = self._free_slots.pop()
        self._requests[request_id] = _Request(slot, len(self.groups))
        self.generation[slot] += 1
        return slot

    def slot_of(self, request_id) -> int:
        return self._req(request_id).slot

    def length(self, request_id) -> int:
        return self._req(request_id).length

    def is_open(self, request_id) -> bool:
        return request_id in self._requests

    def live_requests(self):
        return list(self._requests)

    def _req(self, request_id) -> _Request:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    # ---- pages ---------------------------------------------------------------
    def _first_needed_page(self, g: int, query_pos: int) -> int:
        """Lowest page index that a query at `query_pos` (or any later one) can read in group g."""
        w = self.groups[g].window
        if w is None:
            return 0
        first_key = max(0, query_pos - w + 1)
        return first_key // self.page_size

    def pages_needed(self, request_id, n_new: int) -> List[int]:
        """Pages per group that reserving `n_new` more tokens would take (after releasing
        what the window has passed)."""
        r = self._req(request_id)
        start = r.length + r.reserved
        end = start + n_new
        out = []
        for g in range(len(self.groups)):
            have_upto = -(-start // self.page_size)           # table entries [first_live, have_upto) exist
            want_upto = -(-end // self.page_size)
            first = max(self._first_needed_page(g, start), r.first_live_page[g])
            lo = max(have_upto, first)
            out.append(max(0, want_upto - lo))
        return out

    def free_pages(self) -> List[int]:
        return [p.n_free for p in self.pools]

    def can_reserve(self, request_id, n_new: int) -> bool:
        r = self._req(request_id)
        if r.length + r.reserved + n_new > self.max_pages_per_request * self.page_size:
            return False
        need = self.pages_needed(request_id, n_new)
        # pages that the window lets go before this step count as free
        rel = self._releasable(r, r.length + r.reserved)
        return all(need[g] <= self.pools[g].n_free + rel[g] for g in range(len(self.groups)))

    def _releasable(self, r: _Request, query_pos: int) -> List[int]:
        out = []
        for g in range(len(self.groups)):
            first = self._first_needed_page(g, query_pos)
            held_upto = -(-(r.length + r.reserved) // self.page_size)
            out.append(max(0, min(first, held_upto) - r.first_live_page[g]))
        return out

    def release_behind_window(self, request_id) -> int:
        """Give back the pages no query from position `length` on can read.  Returns how many."""
        r = self._req(request_id)
        n = 0
        for g in range(len(self.groups)):
            first = min(self._first_needed_page(g, r.length + r.reserved),
                        -(-(r.length + r.reserved) // self.page_size))
            tab = self.tables[g][r.slot]
            for i in range(r.first_live_page[g], first):
                if tab[i] >= 0:
                    self.pools[g].give(int(tab[i]))
                    tab[i] = -1
                    n += 1
            r.first_live_page[g] = max(r.first_live_page[g], first)
        return n

    def reserve(self, request_id, n_new: int) -> None:
        """Take the pages that the request's next `n_new` tokens need, in every group, or none."""
        if n_new < 1:
            raise CacheError("reserve needs n_new >= 1")
        r = self._req(request_id)
        start = r.length + r.reserved
        if start + n_new > self.max_pages_per_request * self.page_size:
            raise OutOfPages(f"request {request_id!r} would exceed {self.max_pages_per_request} pages")
        if not self.can_reserve(request_id, n_new):
            raise OutOfPages(f"request {request_id!r}: {self.pages_needed(request_id, n_new)} pages needed, "
                             f"{self.free_pages()} free")
        self.release_behind_window(request_id)
        end = start + n_new
        for g in range(len(self.groups)):
            have_upto = -(-start // self.page_size)
            want_upto = -(-end // self.page_size)
            lo = max(have_upto, r.first_live_page[g])
            tab = self.tables[g][r.slot]
            for i in range(lo, want_upto):
                tab[i] = self.pools[g].take()
            used = self.pools[g].n_pages - self.pools[g].n_free
            self.high_water[g] = max(self.high_water[g], used)
        r.reserved += n_new

    def commit(self, request_id) -> None:
        """The step ran: reserved tokens now count as held."""
        r = self._req(request_id)
        r.length += r.reserved
        r.reserved = 0

    def cancel(self, request_id) -> None:
        """The planned step did not run: give back pages that only the reservation needed."""
        r = self._req(request_id)
        if r.reserved == 0:
            return
        keep_upto = -(-r.length // self.page_size)
        had_upto = -(-(r.length + r.reserved) // self.page_size)
        for g in range(len(self.groups)):
            tab = self.tables[g][r.slot]
            for i in range(max(keep_upto, r.first_live_page[g]), had_upto):
                if tab[i] >= 0:
                    self.pools[g].give(int(tab[i]))
                    tab[i] = -1
        r.reserved = 0

    def close(self, request_id) -> int:
        """The request ended: all its pages and its slot go back.  Returns the slot."""
        r = self._req(request_id)
        upto = -(-(r.length + r.reserved) // self.page_size)
        for g in range(len(self.groups)):
            tab = self.tables[g][r.slot]
            for i in range(r.first_live_page[g], upto):
                if tab[i] >= 0:
                    self.pools[g].give(int(tab[i]))
            tab[:] = -1
        del self._requests[request_id]
        self._free_slots.append(r.slot)
        return r.slot

    def block_table(self, g: int, request_id) -> np.ndarray:
        return self.tables[g][self._req(request_id).slot]

    # ---- checking (tests and debugging) ---------------------------------------
    def audit(self) -> None:
        """Raise if a page is lost, held twice, or a table disagrees with a request's length."""
        for g, pool in enumerate(self.pools):
            seen = np.zeros(pool.n_pages, dtype=np.int32)
            for rid, r in self._requests.items():
                tab = self.tables[g][r.slot]
                upto = -(-(r.length + r.reserved) // self.page_size)
                for i, p in enumerate(tab):
                    if p >= 0:
                        if not (r.first_live_page[g] <= i < upto):
                            raise CacheError(f"group {g} request {rid!r}: page at index {i} outside its live range")
                        seen[p] += 1
                    elif r.first_live_page[g] <= i < upto:
                        raise CacheError(f"group {g} request {rid!r}: hole at index {i}")
            if (seen > 1).any():
                raise CacheError(f"group {g}: page {int(np.argmax(seen > 1))} is in two tables")
            free = np.zeros(pool.n_pages, dtype=np.int32)
            for p in pool._free:
                free[p] += 1
            if (free > 1).any():
                raise CacheError(f"group {g}: page {int(np.argmax(free > 1))} is free twice")
            if ((seen + free) != 1).any():
                bad = int(np.argmax((seen + free) != 1))
                raise CacheError(f"group {g}: page {bad} is {'lost' if seen[bad] + free[bad] == 0 else 'both free and held'}")
            if not (pool._held == (seen == 1)).all():
                raise CacheError(f"group {g}: held flags disagree with the tables")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is used twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")

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

The bookkeeping itself is native code (``csrc/host/page_cache.cpp``, built into
``libxrhost.so`` and called through ctypes); this module gives it its Python
face: requests by id instead of by slot, exceptions instead of return codes.
The block tables are numpy arrays made here and written by the library.  It is
host bookkeeping only (no tensors of keys or values): the device arrays are
owned by the engine.  Nothing is zeroed on reuse; validity is the request's
length.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..csrc import build as _build

_OK, _OUT_OF_PAGES, _TOO_LONG = 0, 1, 2
_host = None


def host_lib() -> ctypes.CDLL:
    """The native host library (compiled at first use; there is no other implementation)."""
    global _host
    if _host is None:
        L = ctypes.CDLL(_build.host_library_path())
        vp, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        sig = {
            "xrh_pool_create": (vp, [i]), "xrh_pool_destroy": (None, [vp]), "xrh_pool_n_free": (i, [vp]),
            "xrh_pool_take": (i, [vp]), "xrh_pool_give": (i, [vp, i]),
            "xrh_cache_create": (vp, [i, vp, i, i, i, i, vp]), "xrh_cache_destroy": (None, [vp]),
            "xrh_has_free_slot": (i, [vp]), "xrh_n_free": (i, [vp, i]), "xrh_high_water": (i, [vp, i]),
            "xrh_pool_take_of": (i, [vp, i]), "xrh_pool_give_of": (i, [vp, i, i]),
            "xrh_open": (i, [vp]), "xrh_close": (i, [vp, i]), "xrh_length": (ll, [vp, i]), "xrh_reserved": (ll, [vp, i]),
            "xrh_pages_needed": (i, [vp, i, ll, vp]), "xrh_can_reserve": (i, [vp, i, ll]), "xrh_reserve": (i, [vp, i, ll]),
            "xrh_commit": (i, [vp, i]), "xrh_cancel": (i, [vp, i]), "xrh_release_behind_window": (i, [vp, i]),
            "xrh_audit": (i, [vp, ctypes.c_char_p, i]),
            "xrh_describe": (ll, [vp, i] + [vp] * 5 + [i, i] + [vp] * 9),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _host = L
    return _host


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
    """A stack of free page numbers with a record of who holds what (a pool on its own)."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError("a pool needs at least one page")
        self.n_pages = n_pages
        self._L = host_lib()
        self._h = self._L.xrh_pool_create(n_pages)
        if not self._h:
            raise MemoryError("the page pool could not be made")

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.xrh_pool_destroy(self._h)
            self._h = None

    @property
    def n_free(self) -> int:
        return self._L.xrh_pool_n_free(self._h)

    def take(self) -> int:
        p = self._L.xrh_pool_take(self._h)
        if p < 0:
            raise OutOfPages("pool is empty")
        return p

    def give(self, page: int) -> None:
        if self._L.xrh_pool_give(self._h, int(page)) != _OK:
            raise CacheError(f"page {page} is given back but not held")


class _GroupPool:
    """One group's pool inside a cache manager."""

    def __init__(self, manager: "CacheManager", g: int, n_pages: int):
        self._m, self._g, self.n_pages = manager, g, n_pages

    @property
    def n_free(self) -> int:
        return self._m._L.xrh_n_free(self._m._h, self._g)

    def take(self) -> int:
        p = self._m._L.xrh_pool_take_of(self._m._h, self._g)
        if p < 0:
            raise OutOfPages("pool is empty")
        return p

    def give(self, page: int) -> None:
        if self._m._L.xrh_pool_give_of(self._m._h, self._g, int(page)) != _OK:
            raise CacheError(f"page {page} is given back but not held")


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
        if n_pages < 1:
            raise CacheError("a pool needs at least one page")
        self.groups = list(groups)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_pages_per_request = -(-max_request_tokens // page_size)
        # block tables: [group][slot, page index] -> page number, -1 where none is held (written by the library)
        self.tables = [np.full((max_requests, self.max_pages_per_request), -1, dtype=np.int32) for _ in self.groups]
        G = len(self.groups)
        self._L = host_lib()
        windows = (ctypes.c_int * max(G, 1))(*[-1 if g.window is None else int(g.window) for g in self.groups])
        self._table_ptrs = (ctypes.c_void_p * max(G, 1))(*[t.ctypes.data for t in self.tables])
        self._h = self._L.xrh_cache_create(G, windows, n_pages, page_size, max_requests, self.max_pages_per_request,
                                           self._table_ptrs)
        if not self._h:
            raise CacheError("the cache manager could not be made (sizes must be positive)")
        self.pools = [_GroupPool(self, g, n_pages) for g in range(G)]
        self._slots: Dict[object, int] = {}                         # request id -> slot
        self.generation = np.zeros(max_requests, dtype=np.int64)   # bumped when a slot is assigned
        self._need = (ctypes.c_int * max(G, 1))()

    def __del__(self):
        if getattr(self, "_h", None):
            self._L.xrh_cache_destroy(self._h)
            self._h = None

    @property
    def high_water(self) -> List[int]:
        return [self._L.xrh_high_water(self._h, g) for g in range(len(self.groups))]

    # ---- requests and slots ------------------------------------------------
    def has_free_slot(self) -> bool:
        return bool(self._L.xrh_has_free_slot(self._h))

    def open(self, request_id) -> int:
        if request_id in self._slots:
            raise CacheError(f"request {request_id!r} is already open")
        slot = self._L.xrh_open(self._h)
        if slot < 0:
            raise OutOfPages("no free request slot")
        self._slots[request_id] = slot
        self.generation[slot] += 1
        return slot

    def slot_of(self, request_id) -> int:
        return self._slot(request_id)

    def length(self, request_id) -> int:
        return self._L.xrh_length(self._h, self._slot(request_id))

    def reserved(self, request_id) -> int:
        """Tokens reserved for a step that has not been committed or cancelled yet."""
        return self._L.xrh_reserved(self._h, self._slot(request_id))

    def is_open(self, request_id) -> bool:
        return request_id in self._slots

    def live_requests(self):
        return list(self._slots)

    def _slot(self, request_id) -> int:
        try:
            return self._slots[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    # ---- pages ---------------------------------------------------------------
    def pages_needed(self, request_id, n_new: int) -> List[int]:
        """Pages per group that reserving `n_new` more tokens would take (after releasing
        what the window has passed)."""
        self._L.xrh_pages_needed(self._h, self._slot(request_id), n_new, self._need)
        return [self._need[g] for g in range(len(self.groups))]

    def free_pages(self) -> List[int]:
        return [self._L.xrh_n_free(self._h, g) for g in range(len(self.groups))]

    def can_reserve(self, request_id, n_new: int) -> bool:
        """Whether `reserve` would succeed; pages that the window lets go before this step count as free."""
        return bool(self._L.xrh_can_reserve(self._h, self._slot(request_id), n_new))

    def release_behind_window(self, request_id) -> int:
        """Give back the pages no query from position `length` on can read.  Returns how many."""
        return self._L.xrh_release_behind_window(self._h, self._slot(request_id))

    def reserve(self, request_id, n_new: int) -> None:
        """Take the pages that the request's next `n_new` tokens need, in every group, or none."""
        if n_new < 1:
            raise CacheError("reserve needs n_new >= 1")
        code = self._L.xrh_reserve(self._h, self._slot(request_id), n_new)
        if code == _TOO_LONG:
            raise OutOfPages(f"request {request_id!r} would exceed {self.max_pages_per_request} pages")
        if code == _OUT_OF_PAGES:
            raise OutOfPages(f"request {request_id!r}: {self.pages_needed(request_id, n_new)} pages needed, "
                             f"{self.free_pages()} free")
        if code != _OK:
            raise CacheError(f"reserve({request_id!r}, {n_new}) failed with code {code}")

    def commit(self, request_id) -> None:
        """The step ran: reserved tokens now count as held."""
        self._L.xrh_commit(self._h, self._slot(request_id))

    def cancel(self, request_id) -> None:
        """The planned step did not run: give back pages that only the reservation needed."""
        self._L.xrh_cancel(self._h, self._slot(request_id))

    def close(self, request_id) -> int:
        """The request ended: all its pages and its slot go back.  Returns the slot."""
        slot = self._slot(request_id)
        self._L.xrh_close(self._h, slot)
        del self._slots[request_id]
        return slot

    def block_table(self, g: int, request_id) -> np.ndarray:
        return self.tables[g][self._slot(request_id)]

    # ---- the step description ---------------------------------------------------
    def describe_step(self, slots: np.ndarray, counts: np.ndarray, tokens: np.ndarray, want_counts: np.ndarray,
                      wants: np.ndarray, fill: int, filler_page: int, out: Sequence[int], block_tables: Sequence[int]) -> int:
        """Flatten a batch into the arrays the kernels read (see ``xrh_describe`` in csrc/host/page_cache.cpp).
        slots, counts, want_counts: int32 per segment; tokens, wants: int32, all segments' one after another;
        out: addresses of the eight int32 arrays (token ids, positions, token -> segment, wanted rows, and per
        segment first row, length, first position, slot); block_tables: one address per group.  Positions are the
        requests' lengths as they are now.  Returns the longest context among the segments."""
        bt = (ctypes.c_void_p * max(len(block_tables), 1))(*block_tables)
        r = self._L.xrh_describe(self._h, len(slots), slots.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
                                 want_counts.ctypes.data, wants.ctypes.data, fill, filler_page, *out, bt)
        if r < 0:
            raise CacheError(f"describe_step: a request of the step is not open (code {r})")
        return int(r)

    # ---- checking (tests and debugging) ---------------------------------------
    def audit(self) -> None:
        """Raise if a page is lost, held twice, or a table disagrees with a request's length."""
        msg = ctypes.create_string_buffer(256)
        if self._L.xrh_audit(self._h, msg, len(msg)) != 0:
            raise CacheError(msg.value.decode())
        slots = list(self._slots.values())
        if len(set(slots)) != len(slots):
            raise CacheError("a request slot is used twice")

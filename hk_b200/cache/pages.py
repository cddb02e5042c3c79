"""Host-side bookkeeping of the paged cache: page pools, block tables, state slots.

The books themselves are C++ (`csrc/runtime.cpp`, built with the C++ compiler at first use); the classes here
are views of those objects: tables and lengths are numpy arrays over the native memory, every decision is made
on the native side.  Nothing here touches the GPU, so every decision can be tested on the CPU.

* A *layer group* is the set of schedule entries whose mixers need the same kind of cache
  (same heads, head size and window).  Each group has a pool of pages and, for every live
  request, a block-table row: logical page i (positions i*page_tokens .. ) -> physical page,
  or -1.  One physical page id addresses the same place in every layer of its group.
* Pages are taken when a request's tokens need them, given back when the request ends and,
  in a windowed group, as soon as the window has passed them; freed pages are reused at once
  (last freed, first reused: stale contents meet new owners early, which the tests want).
* A *state slot* is a request's index into per-request arrays of fixed size: the block-table
  rows and any fixed-size mixer state.  The reference's analogues: a slot per sequence with a
  fixed region (src/cuda/engine.zig:393-401,556-572) and segments grown on demand and freed
  on rewind (src/engine/kv.zig:88-109,137-151).

Errors are returned as exceptions and leave the books unchanged: `OutOfPages`,
`TooManyRequests`, `ContextFull` (cf. `ContextFull`/`NoGpuSlot`, src/engine/model.zig:298,
src/cuda/engine.zig:564).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from ..csrc import build


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


class TooManyRequests(CacheError):
    pass


class ContextFull(CacheError):
    pass


_lib = None


def _runtime() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        lib = build.load("runtime")
        vp, ci = ctypes.c_void_p, ctypes.c_int
        for name, res, args in [
            ("hk_pool_create", vp, [ci]), ("hk_pool_destroy", None, [vp]), ("hk_pool_take", ci, [vp]), ("hk_pool_give", ci, [vp, ci]),
            ("hk_pool_free_count", ci, [vp]), ("hk_pool_num_pages", ci, [vp]), ("hk_pool_held", ctypes.POINTER(ctypes.c_uint8), [vp]),
            ("hk_pool_error", ctypes.c_char_p, [vp]),
            ("hk_books_create", vp, [ctypes.POINTER(ci), ci, ci, ci, ci, ci]), ("hk_books_destroy", None, [vp]),
            ("hk_books_error", ctypes.c_char_p, [vp]), ("hk_books_max_pages", ci, [vp]),
            ("hk_books_length", ctypes.POINTER(ctypes.c_int64), [vp]), ("hk_books_live", ctypes.POINTER(ctypes.c_uint8), [vp]),
            ("hk_books_pool", vp, [vp, ci]), ("hk_books_table", ctypes.POINTER(ctypes.c_int32), [vp, ci]),
            ("hk_books_first_page", ctypes.POINTER(ctypes.c_int32), [vp, ci]), ("hk_books_n_pages", ctypes.POINTER(ctypes.c_int32), [vp, ci]),
            ("hk_books_open", ci, [vp]), ("hk_books_close", ci, [vp, ci]), ("hk_books_release_passed", ci, [vp, ci]),
            ("hk_books_pages_to_take", ci, [vp, ci, ci, ctypes.POINTER(ci)]), ("hk_books_pages_passed", ci, [vp, ci, ctypes.POINTER(ci)]), ("hk_books_free_pages", None, [vp, ctypes.POINTER(ci)]),
            ("hk_books_extend", ci, [vp, ci, ci]), ("hk_books_truncate", ci, [vp, ci, ci]), ("hk_books_audit", ci, [vp]),
        ]:
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


_ERRORS = {-1: OutOfPages, -2: TooManyRequests, -3: ContextFull, -4: CacheError, -5: ValueError}


def _raise(code: int, message: bytes):
    raise _ERRORS.get(code, CacheError)(message.decode())


class PagePool:
    """Free list of page ids 0..num_pages-1 with ownership checks (a view of a native pool: its own, or the
    pool of one layer group of a `CacheBooks`)."""

    def __init__(self, num_pages: int, _handle=None, _owner=None):
        self._rt = _runtime()
        if _handle is None:
            if num_pages < 1:
                raise ValueError("a pool needs at least one page")
            _handle = self._rt.hk_pool_create(int(num_pages))
        self._h = ctypes.c_void_p(_handle)
        self._owner = _owner                 # keeps the books alive; None: this object owns the pool
        self.num_pages = int(self._rt.hk_pool_num_pages(self._h))

    def __del__(self):
        if getattr(self, "_owner", None) is None and getattr(self, "_h", None):
            self._rt.hk_pool_destroy(self._h)
            self._h = None

    @property
    def free_count(self) -> int:
        return int(self._rt.hk_pool_free_count(self._h))

    def take(self) -> int:
        p = self._rt.hk_pool_take(self._h)
        if p < 0:
            _raise(p, self._rt.hk_pool_error(self._h))
        return int(p)

    def give(self, page: int) -> None:
        rc = self._rt.hk_pool_give(self._h, int(page))
        if rc < 0:
            _raise(rc, self._rt.hk_pool_error(self._h))

    def held(self) -> List[int]:
        flags = np.ctypeslib.as_array(self._rt.hk_pool_held(self._h), shape=(self.num_pages,))
        return [int(i) for i in np.nonzero(flags)[0]]


@dataclass
class GroupBooks:
    """One layer group's pool and block table (views of the native books)."""
    window: Optional[int]
    pool: PagePool
    table: np.ndarray            # int32 [max_requests, max_pages_per_request], -1 = none
    first_page: np.ndarray       # int32 [max_requests]: lowest logical page still held
    n_pages: np.ndarray          # int32 [max_requests]: logical pages ever reached (held or passed)


class CacheBooks:
    """Slots, and for each layer group the pages of every live request."""

    def __init__(self, windows: Sequence[Optional[int]], page_tokens: int, num_pages: int, max_requests: int,
                 max_context: int):
        if page_tokens < 1 or max_requests < 1 or max_context < 1:
            raise ValueError("page_tokens, max_requests and max_context must be positive")
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self._rt = rt = _runtime()
        windows = list(windows)
        arr = (ctypes.c_int * max(1, len(windows)))(*[-1 if w is None else int(w) for w in windows])
        self._h = ctypes.c_void_p(rt.hk_books_create(arr, len(windows), int(page_tokens), int(num_pages), int(max_requests),
                                                     int(max_context)))
        if not self._h:
            raise ValueError("the native books refused these sizes")
        self.page_tokens = page_tokens
        self.max_requests = max_requests
        self.max_context = max_context
        self.max_pages_per_request = int(rt.hk_books_max_pages(self._h))
        as_array = np.ctypeslib.as_array
        self.groups: List[GroupBooks] = [
            GroupBooks(w, PagePool(0, _handle=rt.hk_books_pool(self._h, g), _owner=self),
                       as_array(rt.hk_books_table(self._h, g), shape=(max_requests, self.max_pages_per_request)),
                       as_array(rt.hk_books_first_page(self._h, g), shape=(max_requests,)),
                       as_array(rt.hk_books_n_pages(self._h, g), shape=(max_requests,)))
            for g, w in enumerate(windows)]
        self.length = as_array(rt.hk_books_length(self._h), shape=(max_requests,))      # tokens in the cache, per slot
        self.live = as_array(rt.hk_books_live(self._h), shape=(max_requests,)).view(np.bool_)
        self.dirty: set = set()                                 # slots whose table rows changed
        self._take = (ctypes.c_int * max(1, len(windows)))()

    def __del__(self):
        if getattr(self, "_h", None):
            self._rt.hk_books_destroy(self._h)
            self._h = None

    def _check(self, rc: int) -> int:
        if rc < 0:
            _raise(rc, self._rt.hk_books_error(self._h))
        return rc

    # -- slots -----------------------------------------------------------------------------
    def open(self) -> int:
        return self._check(self._rt.hk_books_open(self._h))

    def close(self, slot: int) -> None:
        self._check(self._rt.hk_books_close(self._h, int(slot)))
        self.dirty.add(int(slot))

    # -- pages -----------------------------------------------------------------------------
    def release_passed(self, slot: int) -> int:
        """Gives back the pages of `slot` that its windows have passed; returns how many."""
        n = self._check(self._rt.hk_books_release_passed(self._h, int(slot)))
        if n:
            self.dirty.add(int(slot))
        return n

    def pages_passed(self, slot: int) -> List[int]:
        """For each group: the pages `release_passed(slot)` would give back now."""
        self._check(self._rt.hk_books_pages_passed(self._h, int(slot), self._take))
        return list(self._take[:len(self.groups)])

    def pages_to_take(self, slot: int, n_new: int) -> List[int]:
        """For each group: the pages `extend(slot, n_new)` would take from the pool."""
        self._check(self._rt.hk_books_pages_to_take(self._h, int(slot), int(n_new), self._take))
        return list(self._take[:len(self.groups)])

    def free_pages(self) -> List[int]:
        self._rt.hk_books_free_pages(self._h, self._take)
        return list(self._take[:len(self.groups)])

    def extend(self, slot: int, n_new: int) -> None:
        """Makes room for `n_new` more tokens of `slot`: gives back pages the window has passed,
        then takes the pages the new positions need.  Takes all of them or none."""
        if self._check(self._rt.hk_books_extend(self._h, int(slot), int(n_new))):
            self.dirty.add(int(slot))

    def truncate(self, slot: int, keep: int) -> None:
        """Rewinds `slot` to `keep` tokens, giving back the pages above (cf. src/engine/kv.zig:137-151).
        A windowed group cannot rewind below what it already gave back."""
        self._check(self._rt.hk_books_truncate(self._h, int(slot), int(keep)))
        self.dirty.add(int(slot))

    # -- checks ----------------------------------------------------------------------------
    def audit(self) -> None:
        """Raises if a page is lost, held twice, or free while in a table."""
        self._check(self._rt.hk_books_audit(self._h))

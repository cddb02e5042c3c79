"""Host-side bookkeeping of the paged cache: page pools, block tables, state slots.

Nothing here touches the GPU, so every decision can be tested on the CPU.

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

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


class TooManyRequests(CacheError):
    pass


class ContextFull(CacheError):
    pass


class PagePool:
    """Free list of page ids 0..num_pages-1 with ownership checks."""

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives 0 first
        self._held = np.zeros(num_pages, dtype=bool)

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        if self._held[p]:
            raise CacheError(f"page {p} was on the free list while held")
        self._held[p] = True
        return p

    def give(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise CacheError(f"page {page} is given back but not held")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> List[int]:
        return [int(i) for i in np.nonzero(self._held)[0]]


@dataclass
class GroupBooks:
    """One layer group's pool and block table (host copy)."""
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
        self.page_tokens = page_tokens
        self.max_requests = max_requests
        self.max_context = max_context
        self.max_pages_per_request = -(-max_context // page_tokens)
        self.groups: List[GroupBooks] = [
            GroupBooks(w, PagePool(num_pages),
                       np.full((max_requests, self.max_pages_per_request), -1, dtype=np.int32),
                       np.zeros(max_requests, dtype=np.int32), np.zeros(max_requests, dtype=np.int32))
            for w in windows]
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self.length = np.zeros(max_requests, dtype=np.int64)    # tokens in the cache, per slot
        self.live = np.zeros(max_requests, dtype=bool)
        self.dirty: set = set()                                 # slots whose table rows changed

    # -- slots -----------------------------------------------------------------------------
    def open(self) -> int:
        if not self._free_slots:
            raise TooManyRequests(f"all {self.max_requests} request slots are in use")
        s = self._free_slots.pop()
        self.live[s] = True
        self.length[s] = 0
        for g in self.groups:
            g.first_page[s] = 0
            g.n_pages[s] = 0
        return s

    def close(self, slot: int) -> None:
        self._check_live(slot)
        for g in self.groups:
            for i in range(int(g.first_page[slot]), int(g.n_pages[slot])):
                p = int(g.table[slot, i])
                if p >= 0:
                    g.pool.give(p)
            g.table[slot, :int(g.n_pages[slot])] = -1
            g.first_page[slot] = 0
            g.n_pages[slot] = 0
        self.live[slot] = False
        self.length[slot] = 0
        self.dirty.add(slot)
        self._free_slots.append(slot)

    def _check_live(self, slot: int) -> None:
        if not 0 <= slot < self.max_requests or not self.live[slot]:
            raise CacheError(f"slot {slot} is not live")

    # -- pages -----------------------------------------------------------------------------
    def _passed(self, g: GroupBooks, slot: int, cur: int) -> List[int]:
        """Logical pages of a windowed group that no later token can read: the next query sits at
        position `cur` and reads keys from cur - window + 1 on."""
        if g.window is None:
            return []
        first_needed = max(0, cur - g.window + 1) // self.page_tokens
        return list(range(int(g.first_page[slot]), min(first_needed, int(g.n_pages[slot]))))

    def release_passed(self, slot: int) -> int:
        """Gives back the pages of `slot` that its windows have passed; returns how many."""
        self._check_live(slot)
        cur = int(self.length[slot])
        n = 0
        for g in self.groups:
            for i in self._passed(g, slot, cur):
                g.pool.give(int(g.table[slot, i]))
                g.table[slot, i] = -1
                g.first_page[slot] = i + 1
                n += 1
        if n:
            self.dirty.add(slot)
        return n

    def pages_to_take(self, slot: int, n_new: int) -> List[int]:
        """For each group: the pages `extend(slot, n_new)` would take from the pool."""
        self._check_live(slot)
        want_pages = -(-(int(self.length[slot]) + n_new) // self.page_tokens)
        return [max(0, want_pages - int(g.n_pages[slot])) for g in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.free_count for g in self.groups]

    def extend(self, slot: int, n_new: int) -> None:
        """Makes room for `n_new` more tokens of `slot`: gives back pages the window has passed,
        then takes the pages the new positions need.  Takes all of them or none."""
        self._check_live(slot)
        if n_new < 1:
            raise ValueError("extend needs at least one token")
        cur = int(self.length[slot])
        if cur + n_new > self.max_context:
            raise ContextFull(f"request would reach {cur + n_new} tokens; the context holds {self.max_context}")
        self.release_passed(slot)
        for g, k in zip(self.groups, self.pages_to_take(slot, n_new)):
            if k > g.pool.free_count:
                raise OutOfPages(f"{k} pages needed, {g.pool.free_count} free")
        want_pages = -(-(cur + n_new) // self.page_tokens)
        for g in self.groups:
            for i in range(int(g.n_pages[slot]), want_pages):
                g.table[slot, i] = g.pool.take()
                self.dirty.add(slot)
            g.n_pages[slot] = max(int(g.n_pages[slot]), want_pages)
        self.length[slot] = cur + n_new

    def truncate(self, slot: int, keep: int) -> None:
        """Rewinds `slot` to `keep` tokens, giving back the pages above (cf. src/engine/kv.zig:137-151).
        A windowed group cannot rewind below what it already gave back."""
        self._check_live(slot)
        if not 0 <= keep <= int(self.length[slot]):
            raise ValueError("truncate keeps between 0 and the current length")
        keep_pages = -(-keep // self.page_tokens)
        for g in self.groups:
            if g.window is not None and keep > 0 and max(0, keep - g.window) // self.page_tokens < int(g.first_page[slot]):
                raise CacheError("cannot rewind a windowed cache below pages it has given back")
            for i in range(max(keep_pages, int(g.first_page[slot])), int(g.n_pages[slot])):
                g.pool.give(int(g.table[slot, i]))
                g.table[slot, i] = -1
            g.n_pages[slot] = min(int(g.n_pages[slot]), keep_pages)
            g.first_page[slot] = min(int(g.first_page[slot]), keep_pages)
        self.length[slot] = keep
        self.dirty.add(slot)

    # -- checks ----------------------------------------------------------------------------
    def audit(self) -> None:
        """Raises if a page is lost, held twice, or free while in a table."""
        for gi, g in enumerate(self.groups):
            seen: Dict[int, Tuple[int, int]] = {}
            for s in range(self.max_requests):
                row = g.table[s]
                if not self.live[s]:
                    if (row >= 0).any():
                        raise CacheError(f"group {gi}: dead slot {s} still lists pages")
                    continue
                for i, p in enumerate(row):
                    if p < 0:
                        continue
                    if int(p) in seen:
                        raise CacheError(f"group {gi}: page {int(p)} is held twice ({seen[int(p)]} and {(s, i)})")
                    seen[int(p)] = (s, i)
            held = set(g.pool.held())
            if held != set(seen):
                raise CacheError(f"group {gi}: pool holds {sorted(held - set(seen))} unlisted, tables list {sorted(set(seen) - held)} unheld")
            if len(held) + g.pool.free_count != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.num_pages - len(held) - g.pool.free_count} pages lost")

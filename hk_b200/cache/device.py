"""The cache on the GPU: page tensors, block tables and state arrays, driven by `CacheBooks`.

Layout of a group's pages, per cache of the group: keys [num_pages, n_kv_heads, page_tokens,
k_dim] and values [num_pages, n_kv_heads, page_tokens, v_dim] in the compute type (the two widths
may differ, and a spec with v_dim 0 keeps the key tensor alone), so one (page, kv head) slab of
page_tokens * width elements is contiguous.  (The reference keeps a fixed region
per slot, [layer][kv head][position][head_dim]: src/cuda/engine.zig:234,393-401.)  The block
table of a group is int32 [max_requests, max_pages_per_request] on the device, a copy of the
host books' table; rows that changed are uploaded before a step runs.  A mixer with state of
fixed size gets an array [max_requests, *shape], zeroed when a request takes its slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.base import KVCacheSpec, Precision, StateSpec
from .pages import CacheBooks


@dataclass
class LayerCache:
    """What one schedule entry's mixer is handed."""
    kind: str                                  # "pages" or "state"
    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_tokens: int = 0
    window: Optional[int] = None
    state: Optional[torch.Tensor] = None
    group: int = -1


class PagedCache:
    def __init__(self, cache_specs: Sequence[object], precision: Precision, page_tokens: int, num_pages: int,
                 max_requests: int, max_context: int):
        """`cache_specs`: per schedule entry, the list of specs of the caches its block keeps (a bare spec counts
        as a list of one; None or an empty list: the entry keeps none).  `layers[i]` is the list of `LayerCache`
        that entry's block is handed, in the order of its specs."""
        self.precision = precision
        self.page_tokens = page_tokens
        self.num_pages = num_pages
        entries: List[List[object]] = []
        for spec in cache_specs:
            if spec is None:
                entries.append([])
            elif isinstance(spec, (list, tuple)):
                entries.append([s for s in spec if s is not None])
            else:
                entries.append([spec])
        keys: List[tuple] = []
        for specs in entries:
            for spec in specs:
                if isinstance(spec, KVCacheSpec):
                    key = (spec.n_kv_heads, spec.k_dim, spec.v_dim, spec.window)
                    if key not in keys:
                        keys.append(key)
                elif not isinstance(spec, StateSpec):
                    raise TypeError(f"a cache spec of type {type(spec).__name__}; KVCacheSpec, StateSpec or None are known")
        self.books = CacheBooks([k[3] for k in keys], page_tokens, num_pages, max_requests, max_context)
        dev = precision.device
        self.tables = [torch.full((max_requests, self.books.max_pages_per_request), -1, dtype=torch.int32, device=dev)
                       for _ in keys]
        self.uploaded_bytes = 0
        self.layers: List[List[LayerCache]] = []
        self._states: List[torch.Tensor] = []
        for specs in entries:
            caches: List[LayerCache] = []
            for spec in specs:
                if isinstance(spec, KVCacheSpec):
                    gi = keys.index((spec.n_kv_heads, spec.k_dim, spec.v_dim, spec.window))
                    # zeros, not empty: a page that was never written must not hold NaN patterns
                    k = torch.zeros((num_pages, spec.n_kv_heads, page_tokens, spec.k_dim), dtype=precision.compute, device=dev)
                    v = None
                    if spec.v_dim > 0:
                        v = torch.zeros((num_pages, spec.n_kv_heads, page_tokens, spec.v_dim), dtype=precision.compute, device=dev)
                    caches.append(LayerCache("pages", k, v, self.tables[gi], page_tokens, spec.window, None, gi))
                else:
                    st = torch.zeros((max_requests, *spec.shape), dtype=spec.dtype, device=dev)
                    self._states.append(st)
                    caches.append(LayerCache("state", state=st))
            self.layers.append(caches)

    def has_state(self) -> bool:
        """Whether any mixer keeps a state of fixed size (which running a row twice would advance twice)."""
        return bool(self._states)

    # -- requests ----------------------------------------------------------------------------
    def open(self) -> int:
        slot = self.books.open()
        for st in self._states:
            st[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        self.books.close(slot)

    def sync_tables(self) -> None:
        """Uploads the block-table rows that changed since the last call.  The copies read
        pageable host memory, so they are complete (staged) when the call returns and the
        books may change again at once."""
        if not self.books.dirty:
            return
        for slot in sorted(self.books.dirty):
            for g, dev_table in zip(self.books.groups, self.tables):
                dev_table[slot].copy_(torch.from_numpy(g.table[slot].copy()))
                self.uploaded_bytes += g.table.shape[1] * 4
        self.books.dirty.clear()

    def bytes(self) -> int:
        n = 0
        for caches in self.layers:
            for lc in caches:
                for t in (lc.k_pages, lc.v_pages, lc.state):
                    if t is not None:
                        n += t.numel() * t.element_size()
        return n

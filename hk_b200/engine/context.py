"""What a step hands to the parts: the flattened rows of the batch, who they belong to, and the
host-built tables the parts asked for."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import Part, Precision, StepTables

ALIGN = 8        # int32 elements: every packed array starts on a 32-byte boundary of the buffer


@dataclass
class StepContext:
    """One step's batch, flattened.  Row t is a token; rows of one request are consecutive and
    in increasing position (the reference's rule for items that share a cache:
    src/engine/kv.zig:22-24).

    Device tensors (int32): token_ids[n], positions[n], slot_of_token[n].
    Host lists, one entry per request of the step, in batch order: slots, q_starts (first row),
    q_lens (rows), start_positions (position of the first row).
    `tables[key]` = (device views of the arrays by name, info) for every part that named tables with `key`.
    `fixed_shape`: this step is (or will be replayed as) a captured graph: table shapes and `info` may depend
    only on the number of rows and on `max_context`.  `page_tokens`: the cache's page size.
    """
    precision: Precision
    n_tokens: int
    token_ids: Optional[torch.Tensor]
    positions: Optional[torch.Tensor]
    slot_of_token: Optional[torch.Tensor]
    slots: List[int]
    q_starts: List[int]
    q_lens: List[int]
    start_positions: List[int]
    tables: Dict[Hashable, Tuple[Dict[str, torch.Tensor], object]] = field(default_factory=dict)
    fixed_shape: bool = False
    max_context: int = 0
    page_tokens: int = 0        # tokens per cache page (0: not said); a part may cut its work to fit the pages


def table_parts(model: Part) -> List[Tuple[Hashable, Part]]:
    """The parts of a model that name host-built tables: one (key, part) per distinct key, in the order the
    parts are met.  Found once when a model is built."""
    found: Dict[Hashable, Part] = {}

    def walk(part: Part) -> None:
        key = part.step_tables_key()
        if key is not None and key not in found:
            found[key] = part
        for c in part.children():
            walk(c)

    walk(model)
    return list(found.items())


@dataclass
class PackedStep:
    """A step's integers in one host buffer: [token ids | positions | slots | array | array | ...]; `layout`
    gives, for every key, name -> (offset, shape); `infos` the parts' host-side facts."""
    host: np.ndarray
    layout: Dict[Hashable, Dict[str, Tuple[int, tuple]]]
    infos: Dict[Hashable, object]

    def shape_signature(self):
        return [(k, [(n, off, shp) for n, (off, shp) in arrs.items()]) for k, arrs in self.layout.items()]


def pack_step(meta: np.ndarray, ctx: StepContext, parts: Sequence[Tuple[Hashable, Part]]) -> PackedStep:
    """Asks every table part for its arrays and packs them behind `meta` (int32 [3, n])."""
    pieces = [meta.reshape(-1)]
    cursor = meta.size
    layout: Dict[Hashable, Dict[str, Tuple[int, tuple]]] = {}
    infos: Dict[Hashable, object] = {}
    for key, part in parts:
        st = part.step_tables(ctx)
        if st is None:
            st = StepTables({})
        arrs: Dict[str, Tuple[int, tuple]] = {}
        for name, arr in st.arrays.items():
            a = np.ascontiguousarray(arr, dtype=np.int32)
            pad = -cursor % ALIGN
            if pad:
                pieces.append(np.zeros(pad, dtype=np.int32))
                cursor += pad
            arrs[name] = (cursor, a.shape)
            pieces.append(a.reshape(-1))
            cursor += a.size
        layout[key] = arrs
        infos[key] = st.info
    return PackedStep(np.concatenate(pieces) if len(pieces) > 1 else pieces[0], layout, infos)


def bind_step(ctx: StepContext, packed: PackedStep, device_buffer: torch.Tensor) -> None:
    """Points the context's device tensors and tables at `device_buffer`, which holds (or will hold) `packed.host`."""
    n = ctx.n_tokens
    ctx.token_ids = device_buffer[0:n]
    ctx.positions = device_buffer[n:2 * n]
    ctx.slot_of_token = device_buffer[2 * n:3 * n]
    for key, arrs in packed.layout.items():
        views = {}
        for name, (off, shape) in arrs.items():
            size = int(np.prod(shape)) if len(shape) else 1
            views[name] = device_buffer[off:off + size].view(shape)
        ctx.tables[key] = (views, packed.infos[key])

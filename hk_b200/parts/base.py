"""What every part of a layer has in common, and the registries of part kinds.

A *part* is a piece of a layer that knows its own sizes and constants and nothing about
the model it sits in: a norm, a position encoding, a mixer (attention here), a
feed-forward, a block that arranges them, the embedding, the output head.  A part

  * declares the tensors it needs (`param_specs`: absolute tensor name -> shape and kind),
    which is all the weight loader and the random initialiser know about a model;
  * receives them on the device in its working types (`bind`);
  * runs on the rows of one step (`forward`, signature by part kind, below).

Working types: a `matrix` is held in the compute type (bfloat16 when serving, float32 on the
true 32-bit path), a `vector` (norm weights and the like) always in float32, a `table` of
integers in int32.

Interfaces by kind
  Norm:              forward(x_f32[n, d], out[n, d], rows=None)
  PositionEncoding:  tables() -> (cos, sin, rotary_dim) consumed by the mixer's kernels
  Mixer:             cache_spec() -> KVCacheSpec | StateSpec | None
                     forward(xb[n, d], residual_f32[n, d], ctx, cache, write_cache=True)
                     adds its result onto `residual` in place
  FeedForward:       forward(xb[n, d], residual_f32[n, d], ctx); adds onto `residual` in place
  Block:             cache_specs() -> one spec per cache the block keeps (PreNormBlock: its mixer's)
                     forward(residual_f32[n, d], ctx, caches, write_cache=True); `caches` has one
                     entry per spec, in that order

Host-built tables.  A part that needs small integer tables on the device that depend on the step's
batch (who has how many rows at which positions: work items of a kernel, segment tables of a scan)
does not upload them itself.  It names them with `step_tables_key()` and builds them on the host in
`step_tables(ctx)`; the engine calls that once per step and key (parts with equal keys share the
tables), packs every part's arrays into the one buffer that carries the step's token ids, positions
and slots to the device, and puts the device views into `ctx.tables[key]` before any forward runs.
For a decode step replayed from a captured CUDA graph the engine does the same into the graph's
static buffer; `ctx.fixed_shape` then tells the part that the arrays' shapes may depend only on the
number of rows (and `ctx.max_context`), never on positions.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, Iterable, Optional, Tuple

import numpy as np
import torch

MATRIX, VECTOR, TABLE = "matrix", "vector", "table"


@dataclass(frozen=True)
class ParamSpec:
    shape: Tuple[int, ...]
    kind: str = MATRIX
    init: str = "normal"        # "normal": N(0, std);  "one_plus_normal": 1 + N(0, norm_std)
    optional: bool = False      # absent from the file is not an error (a tied output head)


@dataclass(frozen=True)
class KVCacheSpec:
    """A mixer that keeps keys and values of earlier tokens in pages.
    window: None = all keys stay; w = only the last w positions are ever read again.
    `head_dim` is the width of a key; `v_head_dim` the width of a value when it differs (None: the same;
    0: no value tensor at all, for a mixer that keeps one shared tensor per position)."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None

    @property
    def k_dim(self) -> int:
        return self.head_dim

    @property
    def v_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps a state of fixed size per request (in a state slot)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class StepTables:
    """What `Part.step_tables` returns: int32 arrays by name (any shape), and beside them whatever facts the
    part's forward wants on the host (`info`: counts and sizes that go into kernel launches).  In a step that
    is captured into a CUDA graph, `info` is part of the captured launches: a part must make it a function of
    the batch's shape alone when `ctx.fixed_shape` is set."""
    arrays: Dict[str, np.ndarray]
    info: object = None


class Precision:
    """The engine's working types.  `compute` is torch.bfloat16 or torch.float32."""

    def __init__(self, compute: torch.dtype, device: torch.device):
        if compute not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute type must be bfloat16 or float32, not {compute}")
        self.compute = compute
        self.device = device

    def working_dtype(self, kind: str) -> torch.dtype:
        if kind == MATRIX:
            return self.compute
        if kind == VECTOR:
            return torch.float32
        if kind == TABLE:
            return torch.int32
        raise ValueError(f"unknown parameter kind '{kind}'")


class Part:
    """Base of all parts.  Sub-parts are found through `children()`.

    `graph_safe`: the part's forward reads the step's batch only from the context's device
    tensors and `ctx.tables` (never from its host lists) and launches the same kernels for the same
    batch shape, so a decode step through it can be captured in a CUDA graph.  False unless a part
    says so.  A mixer with a `StateSpec` advances its state every time it runs; the engine therefore
    runs a step exactly once also when it captures it, and fills a batch up with repeated rows (to
    share one graph among batch sizes) only for models that keep no such state: writing the same key
    and value again changes nothing, advancing a state again does."""

    graph_safe = False

    def children(self) -> Iterable["Part"]:
        return ()

    def step_tables_key(self) -> Optional[Hashable]:
        """The name of the host-built tables this part wants in every step, or None (wants none)."""
        return None

    def step_tables(self, ctx) -> Optional["StepTables"]:
        """Builds this step's tables on the host from the context's host lists (`slots`, `q_starts`, `q_lens`,
        `start_positions`).  Called once per step and key."""
        return None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = dict(self.own_param_specs())
        for c in self.children():
            for k, v in c.param_specs().items():
                if k in specs and specs[k] != v:
                    raise ValueError(f"tensor '{k}' is declared twice with different specs")
                specs[k] = v
        return specs

    def own_bind(self, tensors: Dict[str, torch.Tensor], precision: Precision) -> None:
        pass

    def bind(self, tensors: Dict[str, torch.Tensor], precision: Precision) -> None:
        """Takes the declared tensors (device, working types).  A part may fuse or
        re-lay them; it must not keep a reference it does not need."""
        self.own_bind(tensors, precision)
        for c in self.children():
            c.bind(tensors, precision)


# ---- registries of part kinds: name -> class ------------------------------------------

_KINDS: Dict[str, Dict[str, type]] = {"norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}}


def register_part(kind: str, name: str, cls: type) -> None:
    if kind not in _KINDS:
        raise ValueError(f"unknown part kind '{kind}' (kinds: {', '.join(_KINDS)})")
    _KINDS[kind][name] = cls


def part_class(kind: str, name: str) -> type:
    try:
        return _KINDS[kind][name]
    except KeyError:
        raise KeyError(f"no {kind} part named '{name}' (registered: {', '.join(sorted(_KINDS.get(kind, {})))})") from None

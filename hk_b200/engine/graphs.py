"""CUDA graphs for decode steps: one captured forward pass per batch size.

A decode step launches a few hundred small kernels; issued one by one from Python they cost
more than the memory traffic they are bound by (the reference meets the same wall and replays
a graph for passes of up to 8 tokens: src/cuda/engine.zig:772-795).  A `DecodeGraph` captures
the model's forward pass and output head for a batch of B single tokens over *static* device
buffers (token ids, positions, slots, attention work items); a later step copies its own
values into those buffers and replays.  What changes from step to step - which pages, which
positions, how the keys are split - is data in those buffers and in the block tables, never
the graph's shape.  Only models whose parts declare `graph_safe` (they read the batch from
device tensors alone) are captured.
"""
from __future__ import annotations

import gc
from typing import Dict, List

import numpy as np
import torch

from ..csrc import ops
from .context import StepContext


def fill_device_tokens(token_ids, on_device):
    from .engine import fill_device_tokens as fill
    fill(token_ids, on_device)


def graph_batch(n: int) -> int:
    """The batch size of the graph that a decode step of n requests replays: n up to 8, else the next multiple of 8."""
    return n if n <= 8 else -(-n // 8) * 8


class DecodeGraph:
    def __init__(self, engine, batch: int):
        self.engine = engine
        self.batch = batch
        dev = engine.device
        # One static int32 buffer holds everything a step brings: token ids, positions and slots first, then
        # each attention plan's arrays in the order the plans are built.  A replayed step fills a host copy of
        # it and uploads it with ONE copy.
        self.capacity = 3 * batch + 4 * (16 * batch * 8 + 3 * batch)
        self.static = torch.zeros(self.capacity, dtype=torch.int32, device=dev)
        self.meta = self.static[:3 * batch].view(3, batch)
        self.rows = torch.arange(batch, dtype=torch.int32, device=dev)
        self.plan_keys: List[tuple] = []
        self.layout: List[tuple] = []        # (offset, size) of every array after the meta, as captured
        self.graph = None
        self.kernels = 0
        self.logits = None
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self._pending: List[np.ndarray] = []
        self._cursor = 0
        self._immediate = True

    # -- attention plans over the static buffer --------------------------------------------------
    def _splits(self, n_kv_heads: int) -> int:
        # as many CTAs as are resident at once (two per SM), rounded down so that no second, thin wave
        # follows; at most 16 splits, as in the reference (src/cuda/engine.zig:96-101): beyond that the merge of the
        # partials costs more than the split saves
        return max(1, min(16, 2 * self.sms // (self.batch * n_kv_heads)))

    def _upload(self, arr: np.ndarray) -> torch.Tensor:
        """The static region for `arr` (handed out in call order).  While capturing, the values are copied at
        once; on replays they are collected and go up in one copy before the graph is launched."""
        n = arr.size
        off = self._cursor
        if off + n > self.capacity:
            raise RuntimeError("the decode graph's static buffer is too small for this model's attention plans")
        self._cursor = off + n
        region = self.static[off:off + n]
        if self._immediate:
            region.copy_(self.engine.stager.upload(arr).reshape(-1))
            self.layout.append((off, n))
        else:
            self._pending.append(arr.reshape(-1))
        return region.view(arr.shape)

    def _build_plan(self, ctx: StepContext, window: int, n_heads: int, n_kv_heads: int, head_dim: int):
        from ..csrc import attention_fast
        return attention_fast.build_plan(ctx.slots, ctx.q_starts, ctx.q_lens, ctx.start_positions, ctx.n_tokens, window,
                                         n_heads, n_kv_heads, self.sms, self._upload, fixed_splits=self._splits(n_kv_heads),
                                         max_context=self.engine.max_context)

    def _context(self, slots, starts) -> StepContext:
        eng = self.engine
        builder = self._build_plan if eng.plan_builder is not None else None
        b = self.batch
        return StepContext(eng.precision, b, self.meta[0], self.meta[1], self.meta[2], list(slots), list(range(b)),
                           [1] * b, list(starts), plan_builder=builder)

    # -- capture and replay ---------------------------------------------------------------------
    def run(self, meta: np.ndarray, slots, starts, on_device=(), n_real: int = 0) -> torch.Tensor:
        """meta: int32 [3, B] (token ids, positions, slots); `on_device`: (row, DeviceToken) pairs whose ids are
        copied in on the device.  Returns the logits of the first `n_real` rows (all B by default) [n_real, vocab]."""
        eng = self.engine
        ctx = self._context(slots, starts)
        self._cursor = 3 * self.batch
        if self.graph is None:
            self._immediate = True
            self.meta.copy_(eng.stager.upload(meta))
            fill_device_tokens(self.meta[0], on_device)
            # an eager pass first: loads libraries, sets kernel attributes, builds the plans (whose
            # uploads must not be captured); it recomputes this very step, so the cache ends up the same
            x = eng.model.forward(ctx, eng.cache.layers)
            eng.model.head.forward(x, self.rows, self.batch, ctx)
            self.plan_keys = list(ctx.plans.keys())
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            # No cyclic garbage collection while the stream is capturing: it could finalise another engine's graphs,
            # and freeing those is an operation that a capture in progress does not permit.
            gc_was_on = gc.isenabled()
            gc.collect()
            gc.disable()
            try:
                with torch.cuda.graph(graph):
                    x = eng.model.forward(ctx, eng.cache.layers)
                    self.logits = eng.model.head.forward(x, self.rows, self.batch, ctx)
            finally:
                if gc_was_on:
                    gc.enable()
            self.kernels = ops.launch_count() - before      # kernel nodes of the graph
            ops.count_launches(-self.kernels)               # capturing launched nothing
            self.graph = graph
            self._immediate = False
        else:
            self._pending = [meta.reshape(-1)]
            for key in self.plan_keys:
                ctx.attention_plan(*key)      # collects this step's plan arrays, in the captured order
            host = np.concatenate(self._pending)
            if self._cursor != 3 * self.batch + sum(n for _, n in self.layout):
                raise RuntimeError("a decode step's attention plans do not have the captured shape")
            self.static[:host.size].copy_(eng.stager.upload(host))
            fill_device_tokens(self.meta[0], on_device)
        self.graph.replay()
        ops.count_launches(self.kernels)
        return self.logits[:n_real or self.batch].clone()      # the static buffer is overwritten by the next replay


def model_is_graph_safe(model) -> bool:
    def safe(part) -> bool:
        if not getattr(part, "graph_safe", False):
            return False
        return all(safe(c) for c in part.children())
    return all(safe(layer) for layer in model.layers) and safe(model.embedding) and safe(model.head)

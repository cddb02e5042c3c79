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

from typing import Dict, List

import numpy as np
import torch

from ..csrc import ops
from .context import StepContext


class DecodeGraph:
    def __init__(self, engine, batch: int):
        self.engine = engine
        self.batch = batch
        dev = engine.device
        self.meta = torch.zeros((3, batch), dtype=torch.int32, device=dev)
        self.rows = torch.arange(batch, dtype=torch.int32, device=dev)
        self.plan_buffers: Dict[tuple, List[torch.Tensor]] = {}
        self.plan_keys: List[tuple] = []
        self.graph = None
        self.kernels = 0
        self.logits = None
        self.ctx = None
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.sms = sms

    # -- attention plans over static buffers ---------------------------------------------------
    def _splits(self, n_kv_heads: int) -> int:
        # as many CTAs as are resident at once (two per SM), rounded down so that no second, thin wave
        # follows; at most 32 splits (the reference stops at 16: src/cuda/engine.zig:96-101)
        return max(1, min(32, 2 * self.sms // (self.batch * n_kv_heads)))

    def _build_plan(self, ctx: StepContext, window: int, n_heads: int, n_kv_heads: int, head_dim: int):
        from ..csrc import attention_fast
        key = (window, n_heads, n_kv_heads, head_dim)
        bufs = self.plan_buffers.setdefault(key, [])
        idx = [0]

        def upload(arr: np.ndarray) -> torch.Tensor:
            i = idx[0]
            idx[0] += 1
            src = self.engine.stager.upload(arr)
            if i == len(bufs):
                bufs.append(torch.empty_like(src))
            bufs[i].copy_(src)
            return bufs[i]

        return attention_fast.build_plan(ctx.slots, ctx.q_starts, ctx.q_lens, ctx.start_positions, ctx.n_tokens, window,
                                         n_heads, n_kv_heads, self.sms, upload, fixed_splits=self._splits(n_kv_heads),
                                         max_context=self.engine.max_context)

    def _context(self, slots, starts) -> StepContext:
        eng = self.engine
        builder = self._build_plan if eng.plan_builder is not None else None
        b = self.batch
        return StepContext(eng.precision, b, self.meta[0], self.meta[1], self.meta[2], list(slots), list(range(b)),
                           [1] * b, list(starts), plan_builder=builder)

    # -- capture and replay ---------------------------------------------------------------------
    def run(self, meta: np.ndarray, slots, starts) -> torch.Tensor:
        """meta: int32 [3, B] (token ids, positions, slots).  Returns the logits [B, vocab]."""
        eng = self.engine
        self.meta.copy_(eng.stager.upload(meta))
        ctx = self._context(slots, starts)
        if self.graph is None:
            # an eager pass first: loads libraries, sets kernel attributes, builds the plans (whose
            # uploads must not be captured); it recomputes this very step, so the cache ends up the same
            x = eng.model.forward(ctx, eng.cache.layers)
            eng.model.head.forward(x, self.rows, self.batch, ctx)
            self.plan_keys = list(ctx.plans.keys())
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(graph):
                x = eng.model.forward(ctx, eng.cache.layers)
                self.logits = eng.model.head.forward(x, self.rows, self.batch, ctx)
            self.kernels = ops.launch_count() - before      # kernel nodes of the graph
            ops.count_launches(-self.kernels)               # capturing launched nothing
            self.graph = graph
            self.ctx = ctx
        else:
            for key in self.plan_keys:
                ctx.attention_plan(*key)      # refills the static buffers for this step
        self.graph.replay()
        ops.count_launches(self.kernels)
        return self.logits.clone()      # the static buffer is overwritten by the next replay


def model_is_graph_safe(model) -> bool:
    def safe(part) -> bool:
        if not getattr(part, "graph_safe", False):
            return False
        return all(safe(c) for c in part.children())
    return all(safe(layer) for layer in model.layers) and safe(model.embedding) and safe(model.head)

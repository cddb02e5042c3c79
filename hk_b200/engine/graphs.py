"""CUDA graphs for decode steps: one captured forward pass per batch size.

A decode step launches a few hundred small kernels; issued one by one from Python they cost
more than the memory traffic they are bound by (the reference meets the same wall and replays
a graph for passes of up to 8 tokens: src/cuda/engine.zig:772-795).  A `DecodeGraph` captures
the model's forward pass and output head for a batch of B single tokens over ONE static int32
device buffer that holds everything a step brings: token ids, positions and slots, then the
host-built tables of every part that asked for some (`Part.step_tables`).  A later step packs
its own values into a host copy of that buffer, uploads it with one copy and replays.  What
changes from step to step - which pages, which positions, how a part cuts its work - is data
in that buffer and in the block tables, never the graph's shape: parts are told so
(`ctx.fixed_shape`) and the packed layout of every replay is checked against the captured one.
Only models whose parts declare `graph_safe` are captured.

The step that captures runs eagerly, once (the capture itself executes nothing), so a part
that advances per-request state sees every step exactly once.
"""
from __future__ import annotations

import gc

import numpy as np
import torch

from ..csrc import ops
from .context import StepContext, bind_step, pack_step


def graph_batch(n: int) -> int:
    """The batch size of the graph that a decode step of n requests replays: n up to 8, else the next multiple of 8."""
    return n if n <= 8 else -(-n // 8) * 8


class DecodeGraph:
    def __init__(self, engine, batch: int):
        self.engine = engine
        self.batch = batch
        self.rows = torch.arange(batch, dtype=torch.int32, device=engine.device)
        self.static = None              # the step's integers on the device, sized at capture
        self.signature = None           # the packed layout the graph was captured with
        self.graph = None
        self.kernels = 0
        self.logits = None

    def _context(self, slots, starts) -> StepContext:
        eng = self.engine
        b = self.batch
        return StepContext(eng.precision, b, None, None, None, list(slots), list(range(b)), [1] * b, list(starts),
                           fixed_shape=True, max_context=eng.max_context, page_tokens=eng.cache.page_tokens)

    def run(self, meta: np.ndarray, slots, starts, on_device=(), n_real: int = 0) -> torch.Tensor:
        """meta: int32 [3, B] (token ids, positions, slots); `on_device`: (row, DeviceToken) pairs whose ids are
        copied in on the device.  Returns the logits of the first `n_real` rows (all B by default) [n_real, vocab]."""
        eng = self.engine
        ctx = self._context(slots, starts)
        packed = pack_step(meta, ctx, eng._table_parts)
        n_real = n_real or self.batch
        if self.graph is None:
            self.static = torch.zeros(packed.host.size, dtype=torch.int32, device=eng.device)
            self.signature = packed.shape_signature()
            self.static.copy_(eng.stager.upload(packed.host))
            bind_step(ctx, packed, self.static)
            from .engine import fill_device_tokens
            fill_device_tokens(ctx.token_ids, on_device)
            # this step itself runs eagerly: it loads libraries and sets kernel attributes, which a capture
            # must not do, and it is the one execution of the step
            x = eng.model.forward(ctx, eng.cache.layers)
            logits = eng.model.head.forward(x, self.rows, self.batch, ctx)
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
            return logits[:n_real]
        if packed.shape_signature() != self.signature:
            raise RuntimeError("a decode step's host-built tables do not have the shape the graph was captured with "
                               "(a part's step_tables must depend on the batch's shape alone when ctx.fixed_shape is set)")
        self.static.copy_(eng.stager.upload(packed.host))
        from .engine import fill_device_tokens
        fill_device_tokens(self.static[:self.batch], on_device)
        self.graph.replay()
        ops.count_launches(self.kernels)
        return self.logits[:n_real].clone()      # the static buffer is overwritten by the next replay


def model_is_graph_safe(model) -> bool:
    def safe(part) -> bool:
        if not getattr(part, "graph_safe", False):
            return False
        return all(safe(c) for c in part.children())
    return all(safe(layer) for layer in model.layers) and safe(model.embedding) and safe(model.head)

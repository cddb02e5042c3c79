"""A model as data: parts, and the order in which the layers run.

`ModelSpec` holds the embedding, a list of blocks, the output head and a *schedule*: the
list of layer calls of one forward pass.  A call names a layer of the list; the same layer
may be named twice (shared weights, a cache of its own for each call), and a call may read
the cache of an earlier call instead of keeping one (`cache_of`).  The default schedule
runs every layer once in order, which is the reference's loop
(src/engine/cpu_backend.zig:258).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..parts.base import Part


@dataclass(frozen=True)
class LayerCall:
    layer: int
    cache_of: Optional[int] = None   # index (in the schedule) of an earlier call whose cache is read


class ModelSpec(Part):
    def __init__(self, config, embedding, layers: Sequence[Part], head, schedule: Optional[List[LayerCall]] = None):
        self.config = config
        self.embedding = embedding
        self.layers = list(layers)
        self.head = head
        self.schedule = list(schedule) if schedule is not None else [LayerCall(i) for i in range(len(self.layers))]
        for ci, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule entry {ci} names layer {call.layer}, which does not exist")
            if call.cache_of is not None:
                if not 0 <= call.cache_of < ci or self.schedule[call.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {ci} must read the cache of an earlier entry that keeps one")

    def children(self):
        return (self.embedding, *self.layers, self.head)

    @property
    def hidden(self) -> int:
        return self.embedding.hidden

    @property
    def vocab(self) -> int:
        return self.head.vocab

    def cache_specs(self):
        """For each schedule entry: the specs of the caches its block keeps (a list, as the block gives it), or
        None for an entry that keeps none and reads another entry's."""
        out = []
        for call in self.schedule:
            if call.cache_of is not None:
                out.append(None)
            else:
                out.append(list(self.layers[call.layer].cache_specs()))
        return out

    def forward(self, ctx, caches) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns the float32 residual [n, hidden]."""
        x = torch.empty((ctx.n_tokens, self.hidden), dtype=torch.float32, device=ctx.token_ids.device)
        self.embedding.forward(ctx.token_ids, x)
        for ci, call in enumerate(self.schedule):
            own = call.cache_of is None
            self.layers[call.layer].forward(x, ctx, caches[ci if own else call.cache_of], write_cache=own)
        return x

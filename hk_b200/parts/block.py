"""Arrangement of a layer's parts.  `PreNormBlock` is the reference's layer
(src/engine/cpu_backend.zig:258-325): norm -> mixer -> residual sum -> norm -> feed-forward
-> residual sum.  The residual stream is float32; the mixer and the feed-forward add onto
it in place.  A block says which caches it keeps (`cache_specs()`, here the one of its mixer)
and is handed exactly those, so a block with two mixers, or with none, is a block like any other."""
from __future__ import annotations

import torch

from .base import Part, register_part


class PreNormBlock(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, mixer_norm, mixer, ffn_norm, feed_forward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward = mixer_norm, mixer, ffn_norm, feed_forward

    def children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def cache_specs(self):
        """One cache: the mixer's."""
        return [self.mixer.cache_spec()]

    def forward(self, residual: torch.Tensor, ctx, caches, write_cache: bool = True) -> None:
        xb = torch.empty(residual.shape, dtype=ctx.precision.compute, device=residual.device)
        self.mixer_norm.forward(residual, xb)
        self.mixer.forward(xb, residual, ctx, caches[0], write_cache)
        self.ffn_norm.forward(residual, xb)
        self.feed_forward.forward(xb, residual, ctx)


register_part("block", "pre_norm", PreNormBlock)

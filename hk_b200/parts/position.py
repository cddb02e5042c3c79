"""Rotary position encoding: tables of cos and sin by position.

inv_freq[i] = theta^(-2i/rotary_dim) is derived in float64 and cast to float32; the angle
is float32(pos) * inv_freq[i] in float32 (src/engine/ops.zig:96-144,154-161).  cos and sin of
that float32 angle are taken in float64 and rounded once.  Pairing is rotate-half: dims
(i, i + rotary_dim/2) (src/engine/ops.zig:176-181).  theta, the rotary width and the number
of positions are parameters; the tables are shared by every layer that is given this part.
"""
from __future__ import annotations

import torch

from .base import Part, Precision, register_part


class RotaryEmbedding(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, theta: float, rotary_dim: int, max_positions: int):
        if rotary_dim % 2 or rotary_dim < 2:
            raise ValueError(f"rotary width {rotary_dim} must be even and at least 2")
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim)
        self.max_positions = int(max_positions)
        self.cos = None
        self.sin = None

    def inv_freq(self) -> torch.Tensor:
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64), -(2.0 * i) / self.rotary_dim).to(torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        if self.cos is not None:
            return
        pos = torch.arange(self.max_positions, dtype=torch.float32)[:, None]
        angle = (pos * self.inv_freq()[None, :]).to(torch.float32).to(torch.float64)
        self.cos = torch.cos(angle).to(torch.float32).contiguous().to(precision.device)
        self.sin = torch.sin(angle).to(torch.float32).contiguous().to(precision.device)

    def tables(self):
        return self.cos, self.sin, self.rotary_dim


register_part("position", "rope", RotaryEmbedding)

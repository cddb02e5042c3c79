"""RMS norm: out = x * rsqrt(mean(x^2) + eps) * weight, in float32
(src/engine/ops.zig:10-29).  Width, eps, the tensor name and an offset added to the stored weight
(0 here; 1 for checkpoints that store weight - 1) are parameters."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import VECTOR, ParamSpec, Part, Precision, register_part


class RMSNorm(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, width: int, eps: float, weight_name: str, weight_offset: float = 0.0):
        self.width = width
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight_offset = float(weight_offset)
        self.weight: Optional[torch.Tensor] = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        return {self.weight_name: ParamSpec((self.width,), VECTOR, "one_plus_normal")}

    def own_bind(self, tensors, precision: Precision) -> None:
        self.weight = tensors[self.weight_name]
        if self.weight_offset != 0.0:
            self.weight = (self.weight + self.weight_offset).contiguous()     # folded in once; the kernel is the same

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        ops.rms_norm(x, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)

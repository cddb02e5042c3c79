"""SwiGLU feed-forward: residual += (silu(xb Wg^T) * (xb Wu^T)) Wd^T, no biases
(src/engine/cpu_backend.zig:308-323, src/engine/ops.zig:65-80).  Gate and up are one
product over the concatenated weight [2F, d] (the reference fuses them into one parallel
region: src/engine/matmul.zig:93-96)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import MATRIX, ParamSpec, Part, Precision, register_part


class SwiGLUFeedForward(Part):
    def __init__(self, hidden: int, intermediate: int, prefix: str):
        self.hidden, self.F, self.prefix = hidden, intermediate, prefix
        self.w_gate_up = self.w_down = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p = self.prefix
        return {
            p + "gate_proj.weight": ParamSpec((self.F, self.hidden), MATRIX),
            p + "up_proj.weight": ParamSpec((self.F, self.hidden), MATRIX),
            p + "down_proj.weight": ParamSpec((self.hidden, self.F), MATRIX),
        }

    def own_bind(self, tensors, precision: Precision) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        n = xb.shape[0]
        gate_up = torch.empty((n, 2 * self.F), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_gate_up, gate_up)
        h = torch.empty((n, self.F), dtype=xb.dtype, device=xb.device)
        ops.swiglu(gate_up, h)
        ops.gemm(h, self.w_down, residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)

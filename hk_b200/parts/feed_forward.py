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
    graph_safe = True   # reads the batch from device tensors only

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
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        # One matrix [all gate rows | all up rows]: one product gives both halves, and the tensor-core kernels take a
        # tile's rows half from each so that SwiGLU runs in their epilogue (cf. the reference's fused gate/up product,
        # shaders/swiglu_pair.comp:2).
        if gate.dtype != up.dtype:                  # one of them kept in 32-bit: both are
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        h = torch.empty((xb.shape[0], self.F), dtype=xb.dtype, device=xb.device)
        ops.gemm_swiglu(xb, self.w_gate_up, h)
        ops.gemm(h, self.w_down, residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)

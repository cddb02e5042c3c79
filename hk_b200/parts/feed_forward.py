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
        self.block = 0

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
        # Serving layout: rows in blocks of 128 gates followed by their 128 ups, so that one output tile
        # of the tensor-core product holds both halves and SwiGLU runs in its epilogue
        # (cf. the interleaved gate/up of shaders/swiglu_pair.comp:2).  Otherwise [all gates | all ups].
        from ..csrc import gemm_fast
        if gate.dtype != up.dtype:                  # one of them kept in 32-bit: both are
            gate, up = gate.float(), up.float()
        if gate.dtype == torch.bfloat16 and self.F % gemm_fast.PAIR == 0:
            self.block = gemm_fast.PAIR
            self.w_gate_up = gemm_fast.pair_gate_up(gate, up)
        else:
            self.block = 0
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        h = torch.empty((xb.shape[0], self.F), dtype=xb.dtype, device=xb.device)
        ops.gemm_swiglu(xb, self.w_gate_up, h, self.block)
        ops.gemm(h, self.w_down, residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)

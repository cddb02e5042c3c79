"""Token embedding and output head.

Embedding: x[t, :] = E[token_t, :] widened to the float32 residual
(src/engine/cpu_backend.zig:237-244).  Head: final norm on the wanted rows only, then
logits = xb W_out^T in float32 (cpu_backend.zig:329-357); W_out is `lm_head.weight` when
the file has it, else the embedding table when the configuration ties them
(src/engine/weights.zig:124-129; src/convert/hf.zig:313,481-484)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import MATRIX, ParamSpec, Part, Precision


class TokenEmbedding(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, vocab: int, hidden: int, name: str):
        self.vocab, self.hidden, self.name = vocab, hidden, name
        self.table = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.vocab, self.hidden), MATRIX)}

    def own_bind(self, tensors, precision: Precision) -> None:
        self.table = tensors[self.name]

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embedding(self.table, token_ids, out)


class OutputHead(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, vocab: int, norm, name: str, tied_to: Optional[str] = None):
        self.hidden, self.vocab, self.norm, self.name, self.tied_to = hidden, vocab, norm, name, tied_to
        self.weight = None

    def children(self):
        return (self.norm,)

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.vocab, self.hidden), MATRIX, optional=self.tied_to is not None)}

    def own_bind(self, tensors, precision: Precision) -> None:
        w = tensors.get(self.name)
        if w is None:
            w = tensors[self.tied_to]
        self.weight = w

    def forward(self, residual: torch.Tensor, rows: torch.Tensor, n_rows: int, ctx) -> torch.Tensor:
        """Logits float32 [n_rows, vocab] of the residual rows `rows[:n_rows]`."""
        xb = torch.empty((n_rows, self.hidden), dtype=ctx.precision.compute, device=residual.device)
        self.norm.forward(residual, xb, rows)
        logits = torch.empty((n_rows, self.vocab), dtype=torch.float32, device=residual.device)
        ops.gemm(xb, self.weight, logits)
        return logits

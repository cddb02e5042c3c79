"""What a step hands to the parts: the flattened rows of the batch and who they belong to."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..parts.base import Precision


@dataclass
class StepContext:
    """One step's batch, flattened.  Row t is a token; rows of one request are consecutive and
    in increasing position (the reference's rule for items that share a cache:
    src/engine/kv.zig:22-24).

    Device tensors (int32): token_ids[n], positions[n], slot_of_token[n].
    Host lists, one entry per request of the step, in batch order: slots, q_starts (first row),
    q_lens (rows), start_positions (position of the first row).
    """
    precision: Precision
    n_tokens: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    slot_of_token: torch.Tensor
    slots: List[int]
    q_starts: List[int]
    q_lens: List[int]
    start_positions: List[int]
    plans: Dict[tuple, object] = field(default_factory=dict)
    plan_builder: Optional[object] = None

    def attention_plan(self, window: int, n_heads: int, n_kv_heads: int, head_dim: int):
        """The cut of this batch into work items for the flash attention kernels, built once per step
        and (window, heads, groups, head size); None sends attention to the generic kernel."""
        if self.plan_builder is None:
            return None
        key = (window, n_heads, n_kv_heads, head_dim)
        if key not in self.plans:
            self.plans[key] = self.plan_builder(self, window, n_heads, n_kv_heads, head_dim)
        return self.plans[key]

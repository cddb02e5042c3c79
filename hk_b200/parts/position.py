"""Rotary position encoding: tables of cos and sin by position.

inv_freq[i] = theta^(-2i/rotary_dim) is derived in float64 and cast to float32; the angle
is float32(pos) * inv_freq[i] in float32 (src/engine/ops.zig:96-144,154-161).  cos and sin of
that float32 angle are taken in float64, multiplied by `mscale` and rounded once.

Parameters: theta, the rotary width, the number of positions, the *pairing* of the rotated
dims - "half": (i, i + rotary_dim/2), the reference's `.neox` and what Hugging Face imports
use; "adjacent": (2i, 2i + 1), its `.norm` (src/engine/ops.zig:164-181, style chosen per
architecture: src/engine/config.zig:296-309) - and a *scaling* of the frequencies for contexts
longer than the training context (src/engine/ops.zig:96-151; kinds and their parameters:
src/engine/config.zig:42-62,163-223):
  linear   inv / factor
  llama3   wavelengths shorter than orig_ctx / high_freq_factor keep inv, longer than
           orig_ctx / low_freq_factor take inv / factor, the band between is blended
  yarn     a ramp over the dims between the ones that make beta_fast and beta_slow rotations in
           orig_ctx blends inv (high frequencies) and inv / factor (low); cos and sin are
           multiplied by mscale = attn_factor * (0.1 ln(factor) + 1)
The tables are shared by every layer that is given this part.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .base import Part, Precision, register_part

PAIRINGS = ("half", "adjacent")


@dataclass(frozen=True)
class RopeScaling:
    kind: str = "none"                 # none | linear | llama3 | yarn
    factor: float = 1.0
    orig_ctx: int = 0                  # the context length before scaling (llama3, yarn)
    low_freq_factor: float = 1.0       # llama3
    high_freq_factor: float = 4.0      # llama3
    beta_fast: float = 32.0            # yarn
    beta_slow: float = 1.0             # yarn
    attn_factor: float = 1.0           # yarn

    def __post_init__(self):
        if self.kind not in ("none", "linear", "llama3", "yarn"):
            raise ValueError(f"rope scaling type '{self.kind}' is not supported (supported: none, linear, llama3, yarn)")
        if self.kind == "none":
            return
        if not (self.factor >= 1.0 and math.isfinite(self.factor)):
            raise ValueError(f"rope scaling factor {self.factor} must be at least 1")
        if self.kind != "linear" and self.orig_ctx <= 0:
            raise ValueError("rope scaling needs the original context length")
        if self.kind == "llama3" and not 0 < self.low_freq_factor < self.high_freq_factor:
            raise ValueError(f"llama3 rope scaling needs 0 < low_freq_factor < high_freq_factor, got "
                             f"{self.low_freq_factor} and {self.high_freq_factor}")
        if self.kind == "yarn" and not (self.beta_fast > 0 and self.beta_slow > 0 and self.attn_factor > 0):
            raise ValueError("yarn rope scaling needs positive beta_fast, beta_slow and attn_factor")


class RotaryEmbedding(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, theta: float, rotary_dim: int, max_positions: int, pairing: str = "half",
                 scaling: Optional[RopeScaling] = None):
        if rotary_dim % 2 or rotary_dim < 2:
            raise ValueError(f"rotary width {rotary_dim} must be even and at least 2")
        if pairing not in PAIRINGS:
            raise ValueError(f"pairing '{pairing}' is neither 'half' nor 'adjacent'")
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim)
        self.max_positions = int(max_positions)
        self.pairing = pairing
        self.scaling = scaling if scaling is not None else RopeScaling()
        self.cos = None
        self.sin = None

    def inv_freq(self) -> torch.Tensor:
        """float32 [rotary_dim / 2], every step in float64 (src/engine/ops.zig:96-144)."""
        n, r = self.rotary_dim, self.scaling
        low = high = 0.0
        if r.kind == "yarn":
            def corr(rotations: float) -> float:
                return n * math.log(r.orig_ctx / (rotations * 2.0 * math.pi)) / (2.0 * math.log(self.theta))
            low = max(0.0, math.floor(corr(r.beta_fast)))
            high = min(n - 1.0, math.ceil(corr(r.beta_slow)))
            if low == high:
                high += 0.001
        out = []
        for i in range(n // 2):
            inv = math.pow(self.theta, -(2.0 * i) / n)
            if r.kind == "linear":
                v = inv / r.factor
            elif r.kind == "llama3":
                wavelen = 2.0 * math.pi / inv
                if wavelen < r.orig_ctx / r.high_freq_factor:
                    v = inv
                elif wavelen > r.orig_ctx / r.low_freq_factor:
                    v = inv / r.factor
                else:
                    smooth = (r.orig_ctx / wavelen - r.low_freq_factor) / (r.high_freq_factor - r.low_freq_factor)
                    v = (1.0 - smooth) * inv / r.factor + smooth * inv
            elif r.kind == "yarn":
                ramp = min(1.0, max(0.0, (i - low) / (high - low)))
                keep = 1.0 - ramp          # high-frequency dims (ramp 0) keep the original frequency
                v = (inv / r.factor) * (1.0 - keep) + inv * keep
            else:
                v = inv
            out.append(v)
        return torch.tensor(out, dtype=torch.float64).to(torch.float32)

    def mscale(self) -> float:
        """The factor on every cos and sin; only yarn changes it (src/engine/ops.zig:146-151)."""
        r = self.scaling
        if r.kind != "yarn":
            return 1.0
        return float(torch.tensor(r.attn_factor, dtype=torch.float32) *
                     torch.tensor(1.0 + 0.1 * math.log(r.factor), dtype=torch.float64).to(torch.float32))

    def own_bind(self, tensors, precision: Precision) -> None:
        if self.cos is not None:
            return
        pos = torch.arange(self.max_positions, dtype=torch.float32)[:, None]
        angle = (pos * self.inv_freq()[None, :]).to(torch.float32).to(torch.float64)
        m = self.mscale()
        self.cos = (torch.cos(angle) * m).to(torch.float32).contiguous().to(precision.device)
        self.sin = (torch.sin(angle) * m).to(torch.float32).contiguous().to(precision.device)

    def tables(self):
        return self.cos, self.sin, self.rotary_dim


register_part("position", "rope", RotaryEmbedding)

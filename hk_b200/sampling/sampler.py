"""Sampling parameters and the per-request sampling state; the arithmetic runs on the device.

Names, defaults and meanings are the reference's (`Params`, src/sampler.zig:13-28):
temperature 0.8 (<= 0 picks the most likely token), top_k 40 (0 = no limit, capped at 4096),
top_p 0.95, min_p 0.05, repeat_penalty 1.0 over the last `repeat_last_n` = 64 tokens,
frequency_penalty and presence_penalty 0, seed (0 seeds from the clock), logit_bias.  The
chain's order is penalties -> top-k -> top-p -> min-p -> temperature -> draw
(src/sampler.zig:3-6).  The random stream is this engine's own (a counter-based generator
keyed by the seed and the number of tokens drawn so far), so a request repeats exactly under
the same seed whatever else is in the batch; it does not reproduce Zig's generator.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from ..csrc import ops


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    seed: int = 0
    logit_bias: Sequence[Tuple[int, float]] = ()

    def validate(self) -> None:
        if self.temperature < 0 or self.temperature > 100:
            raise ValueError(f"temperature {self.temperature} must be a number from 0 up (to 100)")
        if self.top_k < 0:
            raise ValueError(f"top_k {self.top_k} must be 0 or more")
        if not 0 <= self.top_p <= 1:
            raise ValueError(f"top_p {self.top_p} must be a number from 0 to 1")
        if not 0 <= self.min_p <= 1:
            raise ValueError(f"min_p {self.min_p} must be a number from 0 to 1")
        if not 0.01 <= self.repeat_penalty <= 100:
            raise ValueError(f"repeat_penalty {self.repeat_penalty} must be a positive number")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0

    @property
    def adjusts_logits(self) -> bool:
        return (self.repeat_penalty != 1.0 or self.frequency_penalty != 0 or self.presence_penalty != 0
                or len(self.logit_bias) > 0)


GREEDY = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0)


@dataclass
class SamplingState:
    """What a request's sampling carries from token to token."""
    params: SamplingParams
    seed: int = 0
    drawn: int = 0
    history: List[int] = field(default_factory=list)

    @classmethod
    def start(cls, params: SamplingParams, prompt: Sequence[int] = ()) -> "SamplingState":
        params.validate()
        seed = params.seed
        if seed == 0:   # the reference seeds from the clock (src/sampler.zig:46-52)
            seed = time.time_ns() & 0x7FFFFFFFFFFFFFFF or 0x9E3779B97F4A7C15
        return cls(params, seed, 0, list(prompt))


class Sampler:
    """Draws one token per row of logits on the device."""

    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, states: Sequence[SamplingState]) -> torch.Tensor:
        """logits: float32 [rows, vocab] on the device (modified in place by penalties).
        Returns int32 [rows] on the device and advances each state's draw counter; the caller records
        the tokens with `accept` once it has read them."""
        rows = logits.shape[0]
        if rows != len(states):
            raise ValueError("one sampling state per row of logits")
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if any(s.params.adjusts_logits for s in states):
            self._adjust(logits, states)
        if all(s.params.greedy for s in states):
            ops.argmax(logits, out)
            for s in states:
                s.drawn += 1
            return out
        f = np.empty((3, rows), dtype=np.float32)
        k = np.empty(rows, dtype=np.int32)
        sc = np.empty((2, rows), dtype=np.int64)
        for i, s in enumerate(states):
            p = s.params
            f[0, i], f[1, i], f[2, i] = p.temperature, p.top_p, p.min_p
            k[i] = p.top_k
            sc[0, i], sc[1, i] = s.seed, s.drawn
        fd = torch.from_numpy(f).to(self.device)
        kd = torch.from_numpy(k).to(self.device)
        scd = torch.from_numpy(sc).to(self.device)
        ops.sample(logits, fd[0], kd, fd[1], fd[2], scd[0], scd[1], out)
        for s in states:
            s.drawn += 1          # the draw is made: the next one uses the next counter, whether or not this token has been read
        return out

    def _adjust(self, logits: torch.Tensor, states: Sequence[SamplingState]) -> None:
        offsets, ids, counts, bias = [0], [], [], []
        rp, fp, pp = [], [], []
        for s in states:
            p = s.params
            entries: Dict[int, List[float]] = {}
            if p.repeat_penalty != 1.0 or p.frequency_penalty != 0 or p.presence_penalty != 0:
                recent = s.history if p.repeat_last_n == 0 else s.history[-p.repeat_last_n:]
                for t in recent:
                    entries.setdefault(int(t), [0, 0.0])[0] += 1
            for tok, b in p.logit_bias:
                entries.setdefault(int(tok), [0, 0.0])[1] += float(b)
            for tok, (c, b) in entries.items():
                ids.append(tok)
                counts.append(min(c, 65535))     # the reference counts in saturating u16
                bias.append(b)
            offsets.append(len(ids))
            rp.append(p.repeat_penalty)
            fp.append(p.frequency_penalty)
            pp.append(p.presence_penalty)
        dev = self.device
        if not ids:
            return
        ops.adjust_logits(
            logits, torch.tensor(offsets, dtype=torch.int32, device=dev), torch.tensor(ids, dtype=torch.int32, device=dev),
            torch.tensor(counts, dtype=torch.int32, device=dev), torch.tensor(bias, dtype=torch.float32, device=dev),
            torch.tensor(rp, dtype=torch.float32, device=dev), torch.tensor(fp, dtype=torch.float32, device=dev),
            torch.tensor(pp, dtype=torch.float32, device=dev))

    @staticmethod
    def accept(state: SamplingState, token: int) -> None:
        """Records a drawn token once the host has read it (the history feeds the penalties)."""
        state.history.append(int(token))

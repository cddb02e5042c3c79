"""The Python entry points, in the manner of the reference's Python package.

  * `generate(model, prompts, ...)`: token ids in, token ids out, through the scheduler.
  * `HKForCausalLM.from_pretrained(dir).generate(input_ids, max_new_tokens=20, temperature=1.0,
    top_k=50)`: the reference's signature and defaults (python/hk/modeling.py:621-664); like
    there the result is the input followed by the new tokens.
  * `NativeHKEngine(dir).forward(tokens, pos)` -> logits after the last token, `forward_step`,
    `reset_cache`, `vocab_size`, `context_size` (python/hk/native.py:2298-2369).
Texts, tokenizers and chat templates are outside this engine: prompts are token ids.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .engine import Engine, StepEntry
from .engine.scheduler import Scheduler
from .sampling import SamplingParams

Prompt = Sequence[int]
SERVING_PAGE_TOKENS = 64      # cache pages of the entry points: one TMA box per key tile of the decode attention (measured faster than 16)


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    seconds: float = 0.0
    steps: int = 0
    preemptions: int = 0
    decode_steps: int = 0          # steps after the last prompt portion: single tokens only
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    h2d_bytes_per_step: float = 0.0
    d2h_bytes_per_step: float = 0.0


def _as_prompts(prompts) -> Tuple[List[List[int]], bool]:
    if isinstance(prompts, torch.Tensor):
        if prompts.dim() == 1:
            return [prompts.tolist()], True
        return [row.tolist() for row in prompts], False
    if isinstance(prompts, np.ndarray):
        return _as_prompts(torch.from_numpy(prompts))
    prompts = list(prompts)
    if prompts and isinstance(prompts[0], (int, np.integer)):
        return [[int(t) for t in prompts]], True
    return [[int(t) for t in p] for p in prompts], False


def generate_with_engine(engine: Engine, prompts, max_new_tokens: int = 20, temperature: float = 1.0,
                         top_k: int = 50, top_p: float = 1.0, min_p: float = 0.0, repeat_penalty: float = 1.0,
                         seed: int = 0, eos_token_ids: Optional[Sequence[int]] = None,
                         prefill_chunk: int = 512, stats: Optional[GenerationStats] = None,
                         run_ahead: bool = True) -> List[List[int]]:
    """Generates up to `max_new_tokens` for every prompt; returns the new tokens per prompt.
    temperature 0 picks the most likely token.  With seed != 0, request i draws from the
    stream of seed + i, so results do not depend on batching.  `run_ahead`: launch a decode step before
    the host has read the previous step's tokens (same tokens, less idle GPU time)."""
    plist, _ = _as_prompts(prompts)
    if eos_token_ids is None:
        eos_token_ids = getattr(engine.config, "eos_token_ids", ())
    sched = Scheduler(engine, prefill_chunk=prefill_chunk, eos_token_ids=eos_token_ids, run_ahead=run_ahead)
    ids = []
    for i, p in enumerate(plist):
        params = SamplingParams(temperature=float(temperature), top_k=int(top_k), top_p=float(top_p), min_p=float(min_p),
                                repeat_penalty=float(repeat_penalty), seed=0 if seed == 0 else seed + i)
        ids.append(sched.submit(p, max_new_tokens, params))
    t0 = time.perf_counter()
    if stats is None:
        done = sched.run()
    else:
        # time the tail of pure decode steps apart: it starts when the last prompt portion is in
        t_dec, dec_steps, dec_tokens, h2d0, d2h0 = None, 0, 0, 0, 0
        while sched.has_work():
            prompt_before = sched.stats.prompt_tokens
            dec_before, steps_before = sched.stats.decode_tokens, sched.stats.steps
            sched.step()
            if sched.stats.prompt_tokens != prompt_before or t_dec is None:
                torch.cuda.synchronize()
                t_dec, dec_steps, dec_tokens = time.perf_counter(), 0, 0
                h2d0 = engine.stager.bytes + engine.cache.uploaded_bytes
                d2h0 = sched.stats.d2h_bytes
            else:
                dec_steps += sched.stats.steps - steps_before      # a call that only reads tokens launches nothing
                dec_tokens += sched.stats.decode_tokens - dec_before
        done = sched.finished
        torch.cuda.synchronize()
        stats.seconds = time.perf_counter() - t0
        stats.decode_steps, stats.decode_tokens = dec_steps, dec_tokens
        stats.decode_seconds = time.perf_counter() - (t_dec or t0)
        if dec_steps:
            stats.h2d_bytes_per_step = (engine.stager.bytes + engine.cache.uploaded_bytes - h2d0) / dec_steps
            stats.d2h_bytes_per_step = (sched.stats.d2h_bytes - d2h0) / dec_steps
        stats.prompt_tokens = sched.stats.prompt_tokens
        stats.generated_tokens = sum(len(done[i].output) for i in ids)
        stats.steps = sched.stats.steps
        stats.preemptions = sched.stats.preemptions
    engine.check_kernel_status()
    return [list(done[i].output) for i in ids]


def generate(model: str, prompts, max_new_tokens: int = 20, temperature: float = 1.0, top_k: int = 50,
             top_p: float = 1.0, min_p: float = 0.0, seed: int = 0, dtype: str = "bfloat16",
             max_tokens: Optional[int] = None, **engine_options) -> List[List[int]]:
    """Loads the model folder `model` and generates for `prompts` (lists of token ids)."""
    plist, _ = _as_prompts(prompts)
    if max_tokens is None:
        max_tokens = sum(-(-(len(p) + max_new_tokens) // 64) * 64 for p in plist)
    engine_options.setdefault("max_requests", max(1, min(len(plist), 64)))
    engine_options.setdefault("page_tokens", SERVING_PAGE_TOKENS)
    engine = Engine(model, dtype=dtype, max_tokens=max_tokens, **engine_options)
    return generate_with_engine(engine, plist, max_new_tokens, temperature, top_k, top_p, min_p, seed=seed)


class HKForCausalLM:
    """A loaded model with the reference's `generate` signature."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.config = engine.config

    @classmethod
    def from_pretrained(cls, model_dir: str, dtype: str = "bfloat16", max_tokens: int = 8192, **engine_options):
        engine_options.setdefault("page_tokens", SERVING_PAGE_TOKENS)
        return cls(Engine(model_dir, dtype=dtype, max_tokens=max_tokens, **engine_options))

    def generate(self, input_ids, max_new_tokens: int = 20, temperature: float = 1.0, top_k: int = 50,
                 top_p: float = 1.0, min_p: float = 0.0, seed: int = 0):
        """Returns the input ids followed by the new tokens: a tensor like the input when the rows
        end up equally long, else a list of lists."""
        plist, single = _as_prompts(input_ids)
        new = generate_with_engine(self.engine, plist, max_new_tokens, temperature, top_k, top_p, min_p, seed=seed)
        full = [p + n for p, n in zip(plist, new)]
        if isinstance(input_ids, torch.Tensor) and len({len(f) for f in full}) == 1:
            out = torch.tensor(full, dtype=input_ids.dtype, device=input_ids.device)
            return out[0] if single and input_ids.dim() == 1 else out
        return full[0] if single else full


class NativeHKEngine:
    """One conversation with explicit positions, as the reference's class of this name."""

    def __init__(self, model_dir: str, dtype: str = "bfloat16", context_size: Optional[int] = None):
        from .config import load_config
        cfg = load_config(model_dir)
        ctx = context_size or min(getattr(cfg, "max_position_embeddings", 8192), 8192)   # src/engine/model.zig:114
        self._engine = Engine(model_dir, config=cfg, dtype=dtype, max_tokens=ctx, page_tokens=SERVING_PAGE_TOKENS, max_requests=1, max_context=ctx,
                              max_batch_tokens=ctx)
        self._open = False

    @property
    def vocab_size(self) -> int:
        return self._engine.vocab

    @property
    def context_size(self) -> int:
        return self._engine.max_context

    def reset_cache(self) -> None:
        if self._open:
            self._engine.close_request(0)
            self._open = False

    def forward(self, tokens: Sequence[int], pos: int = 0) -> np.ndarray:
        """Feeds `tokens` starting at position `pos` and returns the logits after the last one."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("forward needs at least one token")
        if not self._open:
            self._engine.open_request(0)
            self._open = True
        have = self._engine.request_length(0)
        if pos > have:
            raise ValueError(f"position {pos} leaves a gap after the {have} cached tokens")
        if pos < have:
            self._engine.cache.books.truncate(self._engine.slot_of(0), pos)
        logits = self._engine.step([StepEntry(0, tokens, [len(tokens) - 1])])
        out = logits[0].cpu().numpy()
        self._engine.check_kernel_status()
        return out

    def forward_step(self, token: int, pos: int) -> np.ndarray:
        return self.forward([token], pos)

    def close(self) -> None:
        self.reset_cache()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

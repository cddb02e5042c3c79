"""The scheduler above the step function: admits requests, cuts prompts into portions under a
token budget, decodes, finishes and frees.

Decisions, after the reference's scheduler loop (src/server/scheduler.zig:229-312):
  * requests wait in a FIFO queue and are admitted while a request slot is free and the pool
    has pages for their first portion (the reference admits into idle slots: :325-357);
  * a step's budget is `max_batch_tokens`: first one token for every decoding request
    (:248-258), then the rest split equally among the requests still reading their prompt,
    at least one token each (:259-281), here also capped by `prefill_chunk`;
  * the last token of a prompt asks for logits (:278); a sampled token is held as `pending`
    and fed at the next step (:121,250-256,429);
  * a request finishes on an end token, at `max_new_tokens`, when the context is full
    (:381-391,427-428), or when it is cancelled (:240).
When pages run out (the reference has fixed slots and cannot meet this): a prompt portion is
shortened to what fits or waits; if even the decoding requests cannot all get their next
page, the most recently admitted request is preempted - its pages are freed and it goes back
to the head of the queue, to be recomputed from its prompt plus the tokens it has produced -
until the rest fits.  A request that could not finish even alone in the pool is refused at
`submit`, so this always ends.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

import torch

from ..cache.pages import OutOfPages
from ..sampling import Sampler, SamplingParams, SamplingState
from .engine import DeviceToken, StepEntry

WAITING, PREFILL, DECODE, FINISHED = "waiting", "prefill", "decode", "finished"


class RequestRefused(ValueError):
    pass


@dataclass
class Request:
    id: int
    prompt: List[int]
    max_new_tokens: int
    sampling: SamplingState
    state: str = WAITING
    fed: int = 0                       # tokens of `tokens()` already in the cache
    output: List[int] = field(default_factory=list)
    pending: Optional[int] = None      # sampled, not yet fed
    finish_reason: Optional[str] = None
    admitted_at: int = -1
    preemptions: int = 0

    def tokens(self) -> List[int]:
        """Everything that has to be in the cache before the next token is sampled, except `pending`."""
        return self.prompt + self.output[:len(self.output) - (1 if self.pending is not None else 0)]


@dataclass
class SchedulerStats:
    steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    d2h_bytes: int = 0
    ahead_steps: int = 0          # decode steps launched before the previous step's tokens were read


@dataclass
class _SampledTokens:
    device: object                 # int32 [n] where the sampler wrote them
    host: object                   # the same in pinned host memory once `event` has passed
    event: object


class Scheduler:
    def __init__(self, engine, sampler=None, max_batch_tokens: Optional[int] = None, prefill_chunk: int = 512,
                 eos_token_ids: Sequence[int] = (), run_ahead: bool = True):
        self.engine = engine
        self.books = engine.cache.books
        self.sampler = sampler if sampler is not None else Sampler(engine.device)
        self.max_batch_tokens = int(max_batch_tokens or engine.max_batch_tokens)
        self.prefill_chunk = int(prefill_chunk)
        self.eos = set(int(t) for t in eos_token_ids)
        self.queue: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[int, Request] = {}
        self.stats = SchedulerStats()
        self.run_ahead = bool(run_ahead)
        self._unread = None            # (requests, their sampled tokens) not read by the host yet
        self._ring = [None] * 4        # pinned buffers with events for the sampled tokens on their way to the host
        self._ring_next = 0
        self._next_id = 0
        self._admissions = 0

    # -- submitting ----------------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], max_new_tokens: int, params: Optional[SamplingParams] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRefused("the prompt has no tokens")
        for t in prompt:
            if not 0 <= t < self.engine.vocab:
                raise RequestRefused(f"token id {t} is outside the vocabulary of {self.engine.vocab}")
        if max_new_tokens < 1:
            raise RequestRefused("max_new_tokens must be at least 1")
        if len(prompt) > self.engine.max_context:
            raise RequestRefused(f"the prompt has {len(prompt)} tokens; the context holds {self.engine.max_context}")
        # the most the request can ever hold: its prompt and all but the last generated token
        most = min(len(prompt) + max_new_tokens - 1, self.engine.max_context)
        pages = -(-most // self.books.page_tokens)
        if any(pages > g.pool.num_pages for g in self.books.groups if g.window is None) or \
                any(min(pages, -(-(g.window + self.max_batch_tokens) // self.books.page_tokens) + 1) > g.pool.num_pages
                    for g in self.books.groups if g.window is not None):
            raise RequestRefused(f"the request needs {pages} pages alone; the pool has fewer")
        req = Request(self._next_id, prompt, int(max_new_tokens),
                      SamplingState.start(params or SamplingParams(), prompt))
        self._next_id += 1
        self.queue.append(req)
        return req.id

    def cancel(self, request_id: int) -> None:
        for r in list(self.queue):
            if r.id == request_id:
                self.queue.remove(r)
                self._finish(r, "cancelled", release=False)
                return
        for r in self.running:
            if r.id == request_id:
                self._finish(r, "cancelled")
                return

    # -- one scheduling step -------------------------------------------------------------------
    def has_work(self) -> bool:
        return bool(self.queue or self.running or self._unread is not None)

    def _pages_for(self, n_tokens: int) -> int:
        return -(-n_tokens // self.books.page_tokens)

    def _admit(self) -> None:
        while self.queue and len(self.running) < self.books.max_requests:
            req = self.queue[0]
            first = min(len(req.tokens()), self.prefill_chunk, self.max_batch_tokens)
            # leave one page for each running request's next decode token
            if min(self.books.free_pages(), default=1 << 30) < self._pages_for(first) + len(self.running):
                if self.running:
                    break
            self.queue.popleft()
            self.engine.open_request(req.id)
            req.state = PREFILL
            req.fed = 0
            req.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(req)

    def _plan(self):
        """[(request, tokens, wants_logits)], decodes first, then prompt portions that fit the
        budget and the free pages.  Returns (plan, short) where `short` says the decodes alone
        do not fit the pool."""
        plan = []
        budget = self.max_batch_tokens
        for r in self.running:
            if r.state == DECODE and budget > 0:
                slot = self.engine.slot_of(r.id)
                self.books.release_passed(slot)
                take = self.books.pages_to_take(slot, 1)
                plan.append((r, [r.pending], True, take))
                budget -= 1
        free = list(self.books.free_pages())
        for *_, take in plan:
            for gi, k in enumerate(take):
                free[gi] -= k
        if any(f < 0 for f in free):
            return plan, True
        prefilling = [r for r in self.running if r.state == PREFILL]
        if prefilling and budget > 0:
            share = max(1, budget // len(prefilling))
            for r in prefilling:
                toks = r.tokens()
                n = min(len(toks) - r.fed, share, self.prefill_chunk, budget)
                slot = self.engine.slot_of(r.id)
                self.books.release_passed(slot)
                # shorten to what the free pages hold, counting the room left in the request's last page
                room = min(free, default=1 << 30) * self.books.page_tokens + (-int(self.books.length[slot])) % self.books.page_tokens
                n = min(n, room)
                if n <= 0:
                    continue
                for gi, k in enumerate(self.books.pages_to_take(slot, n)):
                    free[gi] -= k
                plan.append((r, toks[r.fed:r.fed + n], r.fed + n == len(toks), None))
                budget -= n
        return plan, False

    def _preempt(self, req: Request) -> None:
        self.engine.close_request(req.id)
        self.running.remove(req)
        req.state = WAITING
        req.fed = 0
        req.pending = None          # it becomes an ordinary token of the recomputed prefix
        req.preemptions += 1
        self.stats.preemptions += 1
        self.queue.appendleft(req)

    def _finish(self, req: Request, reason: str, release: bool = True) -> None:
        if release:
            self.engine.close_request(req.id)
            self.running.remove(req)
        req.state = FINISHED
        req.finish_reason = reason
        req.pending = None
        self.finished[req.id] = req
        self.stats.finished += 1

    def step(self) -> List[Request]:
        """One scheduling step: admits, plans, runs one engine step and samples.  Returns the requests
        found finished in this call.

        With `run_ahead`, sampled tokens are left on the device and read one call later: when the next step
        is again pure decoding of the same requests, it is launched first (fed from the device tensor) and
        the host reads the earlier tokens while the GPU already works.  An end token is then seen one step
        late; the extra token computed for that request is dropped with it."""
        done: List[Request] = []
        if self._unread is not None:
            reqs, toks = self._unread
            ahead = self._launch_ahead(reqs, toks) if self._ahead_possible(reqs) else None
            done = self._consume(reqs, toks, fed_already=ahead is not None)
            self._unread = ahead
            if ahead is not None:
                return done
        self._admit()
        while True:
            plan, short = self._plan()
            if not short:
                break
            victim = max(self.running, key=lambda r: r.admitted_at)
            self._preempt(victim)
        if not plan:
            if self.running:
                # nothing fits although requests run: free the newest and try again next step
                self._preempt(max(self.running, key=lambda r: r.admitted_at))
            return done
        entries = [StepEntry(r.id, toks, [len(toks) - 1] if want else []) for r, toks, want, _ in plan]
        logits = self.engine.step(entries)
        self.stats.steps += 1
        wanted = [r for r, _, want, _ in plan if want]
        for r, toks, want, _ in plan:
            if r.state == DECODE:
                r.fed += 1
                r.pending = None
                self.stats.decode_tokens += 1
            else:
                r.fed += len(toks)
                self.stats.prompt_tokens += len(toks)
        if wanted:
            self._unread = (wanted, self._sample(logits, wanted))
            if not self.run_ahead:
                reqs, toks = self._unread
                self._unread = None
                done += self._consume(reqs, toks, fed_already=False)
        return done

    # -- tokens that are sampled but not read yet ------------------------------------------------------
    def _ahead_possible(self, reqs: List[Request]) -> bool:
        """True when the next step can be launched before the unread tokens are known: nothing waits, exactly
        the requests that just sampled keep decoding, none of them can end on a count, none needs its history
        for penalties, and the pool has the pages."""
        if not self.run_ahead or self.queue or len(reqs) != len(self.running):
            return False
        take = [0] * len(self.books.groups)
        for r, q in zip(reqs, self.running):
            if r is not q or r.state != DECODE or r.pending is not None or r.sampling.params.adjusts_logits:
                return False
            total = len(r.prompt) + len(r.output) + 1          # with the unread token
            if len(r.output) + 2 > r.max_new_tokens or total + 1 > self.engine.max_context:
                return False
            slot = self.engine.slot_of(r.id)
            self.books.release_passed(slot)
            for gi, k in enumerate(self.books.pages_to_take(slot, 1)):
                take[gi] += k
        return len(reqs) <= self.max_batch_tokens and all(k <= f for k, f in zip(take, self.books.free_pages()))

    def _launch_ahead(self, reqs: List[Request], toks):
        entries = [StepEntry(r.id, DeviceToken(toks.device, i), [0]) for i, r in enumerate(reqs)]
        logits = self.engine.step(entries)
        self.stats.steps += 1
        self.stats.decode_tokens += len(reqs)
        self.stats.ahead_steps += 1
        for r in reqs:
            r.fed += 1
        return reqs, self._sample(logits, reqs)

    def _sample(self, logits, reqs: List[Request]) -> "_SampledTokens":
        """Samples on the device and starts the copy to the host at once: a copy started later would queue
        behind whatever step is launched in between."""
        toks = self.sampler.sample(logits, [r.sampling for r in reqs])
        if not toks.is_cuda:
            return _SampledTokens(toks, toks, None)
        i = self._ring_next
        self._ring_next = (i + 1) % len(self._ring)
        if self._ring[i] is None or self._ring[i][0].numel() < toks.numel():
            self._ring[i] = (torch.empty(max(64, toks.numel()), dtype=toks.dtype).pin_memory(), torch.cuda.Event())
        host, event = self._ring[i]
        host = host[:toks.numel()]
        host.copy_(toks, non_blocking=True)
        event.record()
        return _SampledTokens(toks, host, event)

    def _consume(self, reqs: List[Request], toks, fed_already: bool) -> List[Request]:
        """Reads sampled tokens from the device and advances their requests."""
        done: List[Request] = []
        if toks.event is not None:
            toks.event.synchronize()
        tokens = toks.host.tolist()
        self.stats.d2h_bytes += 4 * len(tokens)
        for r, tok in zip(reqs, tokens):
            if r.state == FINISHED:                 # ended (an end token, a cancel) while this token was in flight
                continue
            tok = int(tok)
            self.sampler.accept(r.sampling, tok)
            if tok in self.eos:
                self._finish(r, "stop")
                done.append(r)
                continue
            r.output.append(tok)
            if len(r.output) >= r.max_new_tokens:
                self._finish(r, "length")
                done.append(r)
            elif len(r.prompt) + len(r.output) > self.engine.max_context:
                self._finish(r, "context")
                done.append(r)
            else:
                r.pending = None if fed_already else tok
                r.state = DECODE
        return done

    def run(self) -> Dict[int, Request]:
        """Steps until every submitted request has finished."""
        while self.has_work():
            self.step()
        check = getattr(self.engine, "check_kernel_status", None)
        if check is not None:
            check()
        return self.finished

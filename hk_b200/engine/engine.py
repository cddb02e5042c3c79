"""The engine: a model on one GPU, its cache, and the one step function.

`Engine.step(entries)` takes a batch of (request, its next tokens, wanted places): portions
of prompts beside single decoded tokens, cut anywhere.  It runs only those tokens, as one
batch, over the cache that earlier steps left, and returns the float32 logits at the wanted
places.  This is the reference's `forwardItems` + `logitsMany`
(src/engine/model.zig:292-343): a flat list of items mixing sequences, K/V of the whole
batch written before any score is taken (src/engine/cpu_backend.zig:290-295), logits only for the
asked rows (cpu_backend.zig:342-357).  Errors (`BatchTooLarge`, `ContextFull`,
`TokenOutOfRange`, `OutOfPages`; cf. src/engine/model.zig:53-59,296-300) are raised before
anything changes, and the engine stays usable (tests/test_engine.zig:189-203 holds the
reference to the same).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.device import PagedCache
from ..cache.pages import CacheError, ContextFull, OutOfPages
from ..config import ModelConfig, load_config, resolve_architecture
from ..parts.base import Precision
from ..weights.loader import load_tensors, random_tensors
from .context import StepContext, bind_step, pack_step, table_parts


class EngineError(RuntimeError):
    pass


class BatchTooLarge(EngineError):
    pass


class TokenOutOfRange(EngineError):
    pass


class UnknownRequest(EngineError):
    pass


class KernelTimeout(EngineError):
    pass


@dataclass
class DeviceToken:
    """One token id that is still on the device: element `index` of an int32 tensor (a sampler's
    output that the host has not read yet).  It lets the next decode step be launched before the
    host knows the token."""
    tensor: torch.Tensor
    index: int

    def __len__(self) -> int:
        return 1


@dataclass
class StepEntry:
    """A request's share of a step: its next tokens and the places among them (indices into
    `tokens`) whose logits are wanted.  `tokens` is a sequence of ids, or one `DeviceToken`."""
    request: Hashable
    tokens: object
    want: Sequence[int] = ()


_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, torch.bfloat16: torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32, torch.float32: torch.float32,
}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not 'bfloat16' or 'float32'") from None


def _resolve_device(device) -> torch.device:
    if not torch.cuda.is_available():
        raise EngineError("no CUDA device: this engine runs on a GPU only (there is no CPU path)")
    dev = torch.device("cuda", int(device))
    torch.cuda.set_device(dev)
    return dev


def fill_device_tokens(token_ids: torch.Tensor, on_device) -> None:
    """Copies device-resident token ids into their rows of `token_ids` (device to device): runs of consecutive
    rows that take consecutive elements of one tensor go in one copy, repeats of one element in one more."""
    i, n = 0, len(on_device)
    while i < n:
        r0, d0 = on_device[i]
        j = i + 1
        while j < n and on_device[j][1].tensor is d0.tensor and on_device[j][0] == r0 + (j - i) \
                and on_device[j][1].index == d0.index + (j - i):
            j += 1
        if j == i + 1:                     # no run: perhaps the same element again and again (rows that fill a batch up)
            while j < n and on_device[j][1].tensor is d0.tensor and on_device[j][0] == r0 + (j - i) \
                    and on_device[j][1].index == d0.index:
                j += 1
            token_ids[r0:r0 + (j - i)].copy_(d0.tensor[d0.index:d0.index + 1].expand(j - i))
        else:
            token_ids[r0:r0 + (j - i)].copy_(d0.tensor[d0.index:d0.index + (j - i)])
        i = j


class PinnedStager:
    """Host-to-device copies of a step's small integer arrays through pinned memory.

    A ring of pinned buffers, each guarded by an event: a buffer is written again only after
    the copy that last read it has finished, so the copies can be asynchronous."""

    def __init__(self, device: torch.device, slots: int = 4):
        self.device = device
        self.slots = slots
        self._bufs: List[Optional[torch.Tensor]] = [None] * slots
        self._events: List[Optional[torch.cuda.Event]] = [None] * slots
        self._next = 0
        self.bytes = 0

    def upload(self, arr: np.ndarray) -> torch.Tensor:
        """A device int32 tensor with the contents (and shape) of `arr`."""
        i = self._next
        self._next = (i + 1) % self.slots
        n = arr.size
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self._bufs[i] is None or self._bufs[i].numel() < n:
            self._bufs[i] = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
        host = self._bufs[i][:n]
        host.numpy()[:] = arr.reshape(-1)
        dev = host.to(self.device, non_blocking=True)
        if self._events[i] is None:
            self._events[i] = torch.cuda.Event()
        self._events[i].record()
        self.bytes += n * 4
        return dev.view(arr.shape)


class Engine:
    """A model bound to `cuda:device`, with a page pool for `max_tokens` cached tokens."""

    def __init__(self, model_dir: Optional[str] = None, *, config: Optional[ModelConfig] = None,
                 random_seed: Optional[int] = None, random_std: Optional[float] = None,
                 random_norm_std: float = 0.05, random_dtype=None, dtype="bfloat16", max_tokens: int = 8192,
                 page_tokens: int = 16, max_requests: int = 8, max_context: Optional[int] = None,
                 max_batch_tokens: int = 8192, device: int = 0, decode_graphs: bool = True):
        self.device = _resolve_device(device)
        self.precision = Precision(parse_dtype(dtype), self.device)
        if config is None:
            if model_dir is None:
                raise ValueError("give a model folder or a configuration")
            config = load_config(model_dir)
        self.config = config
        _, build_model = resolve_architecture(config.architecture)
        if max_tokens % page_tokens:
            max_tokens += page_tokens - max_tokens % page_tokens
        limit = getattr(config, "max_position_embeddings", None) or max_tokens
        self.max_context = int(max_context) if max_context else int(min(limit, max_tokens))
        self.max_batch_tokens = int(max_batch_tokens)
        # compile, side by side, the kernel libraries this precision runs on (and only those)
        from ..csrc import build as _build
        _build.build_many(_build.libraries_for(self.precision.compute == torch.bfloat16))
        self.model = build_model(config, self.max_context)
        specs = self.model.param_specs()
        with torch.no_grad():
            if random_seed is not None:
                std = random_std if random_std is not None else float(getattr(config, "initializer_range", 0.02))
                # `random_dtype`: the type a model folder of these weights would store its matrices in (they are
                # rounded to it first, then held in the working type): a 32-bit engine with random_dtype bfloat16
                # computes with exactly the matrices of the bfloat16 engine of the same seed
                stored = parse_dtype(random_dtype) if random_dtype is not None else None

                def dtype_of(s):
                    work = self.precision.working_dtype(s.kind)
                    return stored if stored is not None and s.kind == "matrix" and work == torch.float32 else work
                tensors = random_tensors(specs, random_seed, std, random_norm_std, self.device, dtype_of=dtype_of)
                if stored is not None:
                    tensors = {k: v.to(self.precision.working_dtype(specs[k].kind)) for k, v in tensors.items()}
            else:
                tensors = load_tensors(model_dir, specs, self.precision)
            self.model.bind(tensors, self.precision)
            del tensors
        self.cache = PagedCache(self.model.cache_specs(), self.precision, page_tokens, max_tokens // page_tokens,
                                max_requests, self.max_context)
        self.vocab = self.model.vocab
        self._requests: Dict[Hashable, int] = {}
        self.steps_run = 0
        self.stager = PinnedStager(self.device)
        # the word that a timed-out barrier wait inside a tensor-core kernel sets; its value travels to pinned
        # memory after every step, without a synchronisation, and is looked at before the next step
        self._kernel_status = self._kernel_status_host = None
        if self.precision.compute == torch.bfloat16:
            from ..csrc import gemm_fast
            self._kernel_status = gemm_fast.status_flag(self.device)
            self._kernel_status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        # the parts that want host-built tables in every step (one per distinct key), found once
        self._table_parts = table_parts(self.model)
        from .graphs import model_is_graph_safe
        self.decode_graphs = bool(decode_graphs) and model_is_graph_safe(self.model)
        # a batch may be filled up with repeats of its last row only if running a row twice changes nothing:
        # true of key/value pages (the same values are written again), false of a state that is advanced
        self._pad_graphs = not self.cache.has_state()
        self._graphs: Dict[int, object] = {}

    # -- requests ----------------------------------------------------------------------------
    def open_request(self, request: Hashable) -> None:
        if request in self._requests:
            raise EngineError(f"request {request!r} is already open")
        self._requests[request] = self.cache.open()

    def close_request(self, request: Hashable) -> None:
        slot = self._requests.pop(request, None)
        if slot is None:
            raise UnknownRequest(f"request {request!r} is not open")
        self.cache.close(slot)

    def has_request(self, request: Hashable) -> bool:
        return request in self._requests

    def request_length(self, request: Hashable) -> int:
        return int(self.cache.books.length[self.slot_of(request)])

    def slot_of(self, request: Hashable) -> int:
        """The request's slot: its row in the block tables and state arrays."""
        try:
            return self._requests[request]
        except KeyError:
            raise UnknownRequest(f"request {request!r} is not open") from None

    def free_pages(self) -> List[int]:
        return self.cache.books.free_pages()

    # -- the step function -------------------------------------------------------------------
    def check_step(self, entries: Sequence[StepEntry]) -> None:
        """Raises what `step` would raise, changing nothing."""
        books = self.cache.books
        total = 0
        seen = set()
        take = [0] * len(books.groups)
        for e in entries:
            slot = self.slot_of(e.request)
            if e.request in seen:
                raise EngineError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n < 1:
                raise EngineError(f"request {e.request!r} brings no tokens")
            if not isinstance(e.tokens, DeviceToken):       # a sampler's output is inside the vocabulary
                for tok in e.tokens:
                    if not 0 <= int(tok) < self.vocab:
                        raise TokenOutOfRange(f"token id {tok} is outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise EngineError(f"wanted place {w} is outside the {n} tokens of request {e.request!r}")
            if int(books.length[slot]) + n > books.max_context:
                raise ContextFull(
                    f"request {e.request!r} would reach {int(books.length[slot]) + n} tokens; the context holds {books.max_context}")
            total += n
            # pages the window has passed come back before any are taken
            passed = books.pages_passed(slot)
            for gi, k in enumerate(books.pages_to_take(slot, n)):
                take[gi] += k - passed[gi]
        if total > self.max_batch_tokens:
            raise BatchTooLarge(f"{total} tokens in one step; the engine takes {self.max_batch_tokens}")
        for gi, k in enumerate(take):
            if k > books.groups[gi].pool.free_count:
                raise OutOfPages(f"the step needs {k} more pages in group {gi}; {books.groups[gi].pool.free_count} are free")

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns float32 logits [wanted, vocab] on the device, in the order
        of the entries and of their `want`, or None when nothing is wanted."""
        if not entries:
            return None
        self._check_kernel_status()
        self.check_step(entries)
        try:
            return self._run_step(entries)
        finally:
            if self._kernel_status is not None:
                self._kernel_status_host.copy_(self._kernel_status, non_blocking=True)

    def _check_kernel_status(self) -> None:
        if self._kernel_status_host is not None and int(self._kernel_status_host[0]) != 0:
            torch.cuda.synchronize(self.device)
            self._kernel_status.zero_()
            self._kernel_status_host.zero_()
            raise KernelTimeout("a tensor-core kernel gave up waiting on a barrier in an earlier step; "
                                "the logits and the cache since then are invalid")

    def check_kernel_status(self) -> None:
        """Waits for everything launched so far and raises `KernelTimeout` if a kernel of any step gave up a
        bounded wait.  `step` itself looks at the word only when the next step begins and without waiting, so
        whoever hands results to the host after a last step (generation, the replay program, a benchmark)
        calls this first."""
        if self._kernel_status is None:
            return
        torch.cuda.synchronize(self.device)
        self._kernel_status_host[0] = int(self._kernel_status.item())
        self._check_kernel_status()

    def _run_step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        books = self.cache.books
        slots = [self.slot_of(e.request) for e in entries]
        for s in slots:
            books.release_passed(s)
        starts = [int(books.length[s]) for s in slots]
        for s, e in zip(slots, entries):
            books.extend(s, len(e.tokens))
        self.cache.sync_tables()

        n = sum(len(e.tokens) for e in entries)
        meta = np.empty((3, n), dtype=np.int32)
        q_starts, q_lens, rows = [], [], []
        on_device = []                                    # (row, DeviceToken): ids filled in on the device
        r = 0
        for s, st, e in zip(slots, starts, entries):
            m = len(e.tokens)
            if isinstance(e.tokens, DeviceToken):
                meta[0, r] = 0
                on_device.append((r, e.tokens))
            else:
                meta[0, r:r + m] = np.asarray(e.tokens, dtype=np.int32)
            meta[1, r:r + m] = np.arange(st, st + m, dtype=np.int32)
            meta[2, r:r + m] = s
            rows.extend(r + int(w) for w in e.want)
            q_starts.append(r)
            q_lens.append(m)
            r += m
        if self.decode_graphs and n == len(entries) and all(list(e.want) == [0] for e in entries):
            from .graphs import DecodeGraph, graph_batch
            # a graph per batch size would be captured again whenever a request comes or goes; sizes above 8 are
            # rounded up to the next multiple of 8 and the batch is filled with repeats of its last row (the same
            # token at the same place: it writes the same key and value again and its logits are dropped)
            nb = graph_batch(n) if self._pad_graphs else n
            if nb > n:
                meta = np.concatenate([meta, np.repeat(meta[:, -1:], nb - n, axis=1)], axis=1)
                if on_device and on_device[-1][0] == n - 1:
                    on_device += [(r, on_device[-1][1]) for r in range(n, nb)]
                slots = slots + [slots[-1]] * (nb - n)
                starts = starts + [starts[-1]] * (nb - n)
            g = self._graphs.get(nb)
            if g is None:
                g = self._graphs[nb] = DecodeGraph(self, nb)
            self.steps_run += 1
            return g.run(meta, slots, starts, on_device, n)
        ctx = StepContext(self.precision, n, None, None, None, slots, q_starts, q_lens, starts,
                          max_context=self.max_context, page_tokens=self.cache.page_tokens)
        packed = pack_step(meta, ctx, self._table_parts)
        bind_step(ctx, packed, self.stager.upload(packed.host))
        fill_device_tokens(ctx.token_ids, on_device)
        x = self.model.forward(ctx, self.cache.layers)
        self.steps_run += 1
        if not rows:
            return None
        rows_dev = self.stager.upload(np.asarray(rows, dtype=np.int32))
        return self.model.head.forward(x, rows_dev, len(rows), ctx)

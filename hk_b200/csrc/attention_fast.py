"""Plan and launch of the bfloat16 flash attention kernel (`attention_flash.cu`).

A *plan* cuts one step's batch into the kernel's work items for a given (window, heads,
groups): each item is a run of consecutive query tokens of one request and a range of keys.
Runs hold as many tokens as fit the CTA's rows (16 per warp, one row per (token, head of the
group)).  When the batch alone would leave SMs idle (decode: few requests, long contexts),
a run's keys are split among several items; their partial results are merged by the combine
kernel.  The plan depends only on the batch's shape (who has how many tokens at which
positions), never on values.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch

from . import build

_UNSUPPORTED = 100001
TILE_N = 64
MAX_HD = 128


@dataclass
class FlashPlan:
    nw: int                      # warps per CTA
    n_items: int
    items: torch.Tensor          # int32 [n_items, 8] on the device
    n_parts: int                 # partial results in scratch (0: none)
    max_keys: int = 0            # the longest key range of an item
    first: Optional[torch.Tensor] = None   # per token: first partial, number of partials, row within the item
    count: Optional[torch.Tensor] = None
    row0: Optional[torch.Tensor] = None


def supported(hd: int, group: int) -> bool:
    return hd % 16 == 0 and 16 <= hd <= MAX_HD and group <= 64


def tc_prefill_supported(hd: int, group: int) -> bool:
    return hd in (64, 128) and group <= 128


def tc2_prefill_supported(hd: int, group: int, page_tokens: int) -> bool:
    """The tcgen05 kernel with two query tiles per CTA and K/V by TMA: the pages must be whole boxes of a 128-key tile."""
    boxes = (page_tokens % 8 == 0 and 128 % page_tokens == 0) or (page_tokens > 0 and page_tokens % 128 == 0)
    return tc_prefill_supported(hd, group) and boxes


def split_chunk(span: int, want: int) -> int:
    """Keys per split when `span` keys (counted from a tile boundary) go to `want` splits: whole tiles."""
    return -(-(-(-span // want)) // TILE_N) * TILE_N


@dataclass
class PlanInfo:
    """The host-side facts of a plan: what goes into the kernel launches beside the arrays."""
    nw: int
    n_items: int
    n_parts: int
    max_keys: int


def decode_splits(n_rows: int, n_kv_heads: int, sm_count: int) -> int:
    """Key splits per request for a decode batch whose plan must keep its shape from step to step: as many
    CTAs as are resident at once (two per SM), rounded down so that no second, thin wave follows; at most 8
    (the reference allows 16, src/cuda/engine.zig:96-101; measured here at batch 1 to 4 over contexts of 512 to
    8,192, attention and merge together: 8 is the fastest or within a microsecond of it everywhere but at batch 1
    over 8,192 tokens (29.7 us against 26.5 with 16), and 16 costs 8 to 10 us more at batch 3 and 4, since the merge
    of the partials costs more than the finer split saves)."""
    return max(1, min(8, 2 * sm_count // max(1, n_rows * n_kv_heads)))


def plan_arrays(slots, q_starts, q_lens, start_positions, n_tokens: int, window: int, H: int, G: int,
                sm_count: int, fixed_splits: int = 0, max_context: int = 0, prefill_rows: int = 64):
    """The plan on the host: (items int32 [n_items, 8], merge int32 [3, n_tokens] or None, PlanInfo), or None
    when the kernels do not take this grouping.  `fixed_splits` > 0 forces that many items per run (a shape
    that does not change from step to step, for captured decode graphs); `max_context` then bounds the key
    range any later step can bring, which sizes the kernel's page-id buffer.  `prefill_rows`: rows per CTA for
    batches with prompt portions: 64 (the mma.sync kernel), 128 (the tcgen05 kernel, head sizes 64 and 128) or 256
    (its variant with two query tiles per CTA, which also wants TMA-able pages: `tc2_prefill_supported`)."""
    group = H // G
    nw = 1 if all(l == 1 for l in q_lens) else prefill_rows // 16
    rows = 16 * nw
    if group > rows:
        if group > 64:
            return None
        nw, rows = 4, 64
    tpb = rows // group
    if fixed_splits > 0 and nw == 1:
        return _decode_plan(slots, q_starts, start_positions, n_tokens, window, fixed_splits, max_context)
    runs = []
    for slot, qs, ql, p0 in zip(slots, q_starts, q_lens, start_positions):
        for b0 in range(0, ql, tpb):
            n = min(tpb, ql - b0)
            pos0 = p0 + b0
            kv_hi = pos0 + n
            kv_lo = max(0, pos0 - window + 1) if window > 0 else 0
            runs.append((qs + b0, n, slot, pos0, kv_lo, kv_hi))
    if nw != 1:
        # longest key ranges first: the heavy items of a causal prompt (its last rows) must not form the tail
        runs.sort(key=lambda r: r[4] - r[5])
    base_ctas = len(runs) * G
    recs = []
    merge = np.zeros((3, n_tokens), dtype=np.int32)       # per token: first partial, number of partials, row within the item
    n_parts = 0
    for (q_row0, n, slot, pos0, kv_lo, kv_hi) in runs:
        kv_len = kv_hi - kv_lo
        if fixed_splits > 0:
            want = fixed_splits
        elif base_ctas >= 2 * sm_count or nw >= 8:
            want = 1
        else:
            want = max(1, min(2 * sm_count // base_ctas, kv_len // 64, 32))
        # splits start on tile boundaries of absolute key positions, so a tile is never shared; the chunk is
        # sized from that aligned start (at or below kv_lo), so that the last split always reaches kv_hi
        start = (kv_lo // TILE_N) * TILE_N
        chunk = split_chunk(kv_hi - start, want)
        n_split = fixed_splits if fixed_splits > 0 else max(1, -(-(kv_hi - start) // chunk))
        if n_split == 1:
            recs.append((q_row0, n, slot, pos0, kv_lo, kv_hi, -1, 0))
            continue
        for s in range(n_split):
            a = max(kv_lo, start + s * chunk)
            b = min(kv_hi, start + (s + 1) * chunk)
            recs.append((q_row0, n, slot, pos0, a, max(a, b), n_parts + s, 0))
        for tq in range(n):
            merge[:, q_row0 + tq] = (n_parts, n_split, tq * group)
        n_parts += n_split
    items = np.asarray(recs, dtype=np.int32).reshape(-1, 8)
    max_keys = max((r[5] - r[4] for r in recs), default=0)
    if fixed_splits > 0 and max_context > 0:
        max_keys = max(max_keys, -(-max_context // fixed_splits) + 2 * TILE_N)
    return items, (merge if n_parts else None), PlanInfo(nw, len(recs), n_parts, max_keys)


def _decode_plan(slots, q_starts, start_positions, n_tokens, window, splits, max_context):
    """The plan of a batch of single tokens with a fixed number of key splits, in array arithmetic (this runs
    on the host before every replayed decode step).  Same items as the general loop gives."""
    B = len(slots)
    pos = np.asarray(start_positions, dtype=np.int64)
    slot = np.asarray(slots, dtype=np.int64)
    qrow = np.asarray(q_starts, dtype=np.int64)
    kv_hi = pos + 1
    kv_lo = np.maximum(0, pos - window + 1) if window > 0 else np.zeros(B, dtype=np.int64)
    kv_len = kv_hi - kv_lo
    max_keys = int(kv_len.max()) if B else 0
    if max_context > 0:
        max_keys = max(max_keys, -(-max_context // splits) + 2 * TILE_N)
    items = np.zeros((B, splits, 8), dtype=np.int32)
    items[:, :, 0] = qrow[:, None]
    items[:, :, 1] = 1
    items[:, :, 2] = slot[:, None]
    items[:, :, 3] = pos[:, None]
    if splits == 1:
        items[:, 0, 4], items[:, 0, 5], items[:, 0, 6] = kv_lo, kv_hi, -1
        return items.reshape(B, 8), None, PlanInfo(1, B, 0, max_keys)
    start = (kv_lo // TILE_N) * TILE_N
    chunk = -(-(-(-(kv_hi - start) // splits)) // TILE_N) * TILE_N     # split_chunk, in array form
    s = np.arange(splits, dtype=np.int64)[None, :]
    a = np.maximum(kv_lo[:, None], start[:, None] + s * chunk[:, None])
    b = np.maximum(a, np.minimum(kv_hi[:, None], start[:, None] + (s + 1) * chunk[:, None]))
    items[:, :, 4], items[:, :, 5] = a, b
    items[:, :, 6] = np.arange(B, dtype=np.int64)[:, None] * splits + s
    merge = np.zeros((3, n_tokens), dtype=np.int32)
    merge[0, qrow] = np.arange(B) * splits
    merge[1, qrow] = splits
    return items.reshape(B * splits, 8), merge, PlanInfo(1, B * splits, B * splits, max_keys)


def plan_on_device(info: PlanInfo, items: torch.Tensor, merge: Optional[torch.Tensor]) -> FlashPlan:
    plan = FlashPlan(info.nw, info.n_items, items, info.n_parts, info.max_keys)
    if info.n_parts:
        plan.first, plan.count, plan.row0 = merge[0], merge[1], merge[2]
    return plan


def build_plan(slots, q_starts, q_lens, start_positions, n_tokens: int, window: int, H: int, G: int,
               sm_count: int, upload: Callable[[np.ndarray], torch.Tensor], fixed_splits: int = 0,
               max_context: int = 0, prefill_rows: int = 64) -> Optional[FlashPlan]:
    """`plan_arrays` followed by `upload(int32 array) -> device tensor` for each array."""
    got = plan_arrays(slots, q_starts, q_lens, start_positions, n_tokens, window, H, G, sm_count, fixed_splits,
                      max_context, prefill_rows)
    if got is None:
        return None
    items, merge, info = got
    return plan_on_device(info, upload(items), upload(merge) if merge is not None else None)


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def tma_decode_supported(hd: int, group: int, page_tokens: int) -> bool:
    return hd in (64, 128) and group <= 16 and page_tokens >= 16 and page_tokens & (page_tokens - 1) == 0


def run(q, k_pages, v_pages, block_table, out, H, G, hd, page_tokens, window, scale, plan: FlashPlan,
        allow_tma: bool = True) -> bool:
    from . import gemm_fast, ops
    if not supported(hd, H // G) or plan is None:
        return False
    lib = build.load("attention_flash")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows = 16 * plan.nw
    part_o = part_ml = None
    if plan.n_parts:
        part_o = torch.empty((plan.n_parts, G, rows, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((plan.n_parts, G, rows, 2), dtype=torch.float32, device=q.device)
    if plan.nw == 16:
        if plan.n_parts or not tc2_prefill_supported(hd, H // G, int(page_tokens)):
            return False
        lib_tc = build.load("attention_prefill_tc")
        code = lib_tc.hk_attention_prefill_tc2(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), ctypes.c_longlong(k_pages.shape[0]), _ptr(block_table),
            int(block_table.shape[1]), _ptr(plan.items), plan.n_items, _ptr(out), H, G, hd, int(page_tokens), int(window),
            ctypes.c_float(scale * math.log2(math.e)), plan.max_keys // int(page_tokens) + 2,
            _ptr(gemm_fast.status_flag(q.device)), stream)
        if code == _UNSUPPORTED:
            return False
        ops._check(code, "paged_attention (tcgen05 prefill, two query tiles)")
        return True
    if plan.nw == 8:
        if plan.n_parts or not tc_prefill_supported(hd, H // G):
            return False
        lib_tc = build.load("attention_prefill_tc")
        code = lib_tc.hk_attention_prefill_tc(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), int(block_table.shape[1]), _ptr(plan.items),
            plan.n_items, _ptr(out), H, G, hd, int(page_tokens), int(window), ctypes.c_float(scale * math.log2(math.e)),
            plan.max_keys // int(page_tokens) + 2, _ptr(gemm_fast.status_flag(q.device)), stream)
        if code == _UNSUPPORTED:
            return False
        ops._check(code, "paged_attention (tcgen05 prefill)")
        return True
    code = _UNSUPPORTED
    if plan.nw == 1 and allow_tma and tma_decode_supported(hd, H // G, int(page_tokens)):
        code = lib.hk_attention_decode_tma(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), ctypes.c_longlong(k_pages.shape[0]), _ptr(block_table),
            int(block_table.shape[1]), _ptr(plan.items), plan.n_items, _ptr(out), _ptr(part_o), _ptr(part_ml), H, G, hd,
            int(page_tokens), int(window), ctypes.c_float(scale * math.log2(math.e)), plan.max_keys // int(page_tokens) + 2,
            _ptr(gemm_fast.status_flag(q.device)), stream)
    if code == _UNSUPPORTED:
        code = lib.hk_attention_flash(_ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), int(block_table.shape[1]),
                                      _ptr(plan.items), plan.n_items, plan.nw, _ptr(out), _ptr(part_o), _ptr(part_ml), H, G, hd,
                                      int(page_tokens), int(window), ctypes.c_float(scale * math.log2(math.e)),
                                      plan.max_keys // int(page_tokens) + 2, stream)
    if code == _UNSUPPORTED:
        return False
    ops._check(code, "paged_attention (flash)")
    if plan.n_parts:
        code = lib.hk_attention_combine(_ptr(part_o), _ptr(part_ml), _ptr(plan.first), _ptr(plan.count), _ptr(plan.row0),
                                        _ptr(out), q.shape[0], H, G, hd, rows, stream)
        ops._check(code, "paged_attention (combine)")
    return True

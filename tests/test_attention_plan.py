"""The cut of a step's attention into work items, checked on the CPU: whatever the window, the
positions and the number of splits, the items of every run of query tokens cover that run's
visible keys [kv_lo, kv_hi) exactly once, in order, without a key left out or read twice."""
import numpy as np
import pytest
import torch

from hk_b200.csrc import attention_fast


def _plan(lens_and_spans, window, H, G, sms=148, fixed_splits=0, prefill_rows=64, max_context=0):
    slots = list(range(len(lens_and_spans)))
    q_starts, q_lens, starts = [], [], []
    r = 0
    for p0, n in lens_and_spans:
        q_starts.append(r)
        q_lens.append(n)
        starts.append(p0)
        r += n
    uploaded = []

    def upload(a):
        uploaded.append(np.array(a))
        return torch.from_numpy(np.ascontiguousarray(a))

    plan = attention_fast.build_plan(slots, q_starts, q_lens, starts, r, window, H, G, sms, upload,
                                     fixed_splits=fixed_splits, max_context=max_context, prefill_rows=prefill_rows)
    return plan, uploaded[0].reshape(-1, 8), r


def _check_cover(items, window, n_tokens):
    """Every run (first query row, tokens, slot, first position) has key ranges that tile [kv_lo, kv_hi)."""
    runs = {}
    for q_row0, n, slot, pos0, a, b, part, _ in items.tolist():
        runs.setdefault((q_row0, n, slot, pos0), []).append((a, b, part))
    seen_rows = set()
    for (q_row0, n, slot, pos0), ranges in runs.items():
        kv_hi = pos0 + n
        kv_lo = max(0, pos0 - window + 1) if window > 0 else 0
        ranges.sort(key=lambda r: (r[2], r[0]))
        cur = kv_lo
        for a, b, part in ranges:
            assert a <= b
            if a == b:
                continue                        # an empty split: merged with weight zero
            assert a == cur, f"run at row {q_row0}: keys {cur}..{a} are left out or read twice"
            cur = b
        assert cur == kv_hi, f"run at row {q_row0}: keys {cur}..{kv_hi} are never read"
        if len(ranges) > 1:
            assert all(p >= 0 for _, _, p in ranges)
        for t in range(n):
            assert q_row0 + t not in seen_rows
            seen_rows.add(q_row0 + t)
    assert seen_rows == set(range(n_tokens))


@pytest.mark.parametrize("window,pos,splits", [
    (100, 133, 2), (128, 133, 0), (128, 190, 2), (1000, 4999, 16), (4096, 5000, 4), (4096, 4097, 16),
    (64, 64, 2), (65, 128, 3), (0, 133, 5), (0, 63, 4), (13, 40, 2)])
def test_split_items_reach_the_newest_key(window, pos, splits):
    plan, items, n = _plan([(pos, 1)], window, 8, 2, sms=4000 if splits == 0 else 148, fixed_splits=splits)
    _check_cover(items, window, n)
    full = items[items[:, 5] > items[:, 4]]
    assert int(full[:, 5].max()) == pos + 1           # the token's own key is in some item


def test_random_batches_are_covered_exactly_once():
    rng = np.random.default_rng(0)
    for trial in range(400):
        window = int(rng.choice([0, 0, 1, 13, 64, 65, 100, 128, 1000, 4096]))
        decode = bool(rng.integers(0, 2))
        n_req = int(rng.integers(1, 9))
        spans = []
        for _ in range(n_req):
            p0 = int(rng.integers(0, 6000))
            spans.append((p0, 1 if decode else int(rng.integers(1, 300))))
        fixed = int(rng.choice([0, 0, 1, 2, 3, 4, 7, 16])) if decode else 0
        sms = int(rng.choice([4, 148, 4000]))
        H, G = [(8, 2), (4, 4), (32, 8), (6, 2)][int(rng.integers(0, 4))]
        rows = int(rng.choice([64, 128]))
        plan, items, n = _plan(spans, window, H, G, sms=sms, fixed_splits=fixed, prefill_rows=rows, max_context=8192)
        _check_cover(items, window, n)
        assert plan.max_keys >= int((items[:, 5] - items[:, 4]).max())
        if fixed > 1:
            assert items.shape[0] == n_req * fixed          # the shape a captured graph relies on


def test_decode_plan_in_array_arithmetic_equals_the_general_loop():
    rng = np.random.default_rng(1)
    for trial in range(100):
        window = int(rng.choice([0, 64, 100, 4096]))
        splits = int(rng.choice([2, 4, 16]))
        B = int(rng.integers(1, 9))
        pos = [int(rng.integers(0, 7000)) for _ in range(B)]
        items, merge, info = attention_fast._decode_plan(list(range(B)), list(range(B)), pos, B, window, splits, 8192)
        items = items.reshape(B, splits, 8)
        for i, p in enumerate(pos):
            kv_hi = p + 1
            kv_lo = max(0, p - window + 1) if window > 0 else 0
            start = kv_lo // 64 * 64
            chunk = attention_fast.split_chunk(kv_hi - start, splits)
            for s in range(splits):
                a = max(kv_lo, start + s * chunk)
                b = max(a, min(kv_hi, start + (s + 1) * chunk))
                assert (int(items[i, s, 4]), int(items[i, s, 5])) == (a, b)
        assert info.n_parts == B * splits and merge.shape == (3, B)


def test_the_attention_part_takes_two_query_tiles_only_when_their_items_fill_the_gpu():
    """The mixer's `step_tables` picks the rows per work item: 256 (two query tiles per CTA) when those items are
    about as many as the SMs, 128 below that, and never where the pages do not suit the TMA boxes."""
    from hk_b200.engine.context import StepContext
    from hk_b200.parts import GQAAttention
    part = GQAAttention(4096, 32, 8, 128, "a.", qk_norm_eps=None, position=None)
    part._sm_count = 148
    part._tables_key = ("attention", 32, 8, 128, 0)

    def rows_per_item(q_lens, page_tokens=16):
        starts = list(np.cumsum([0] + q_lens[:-1]))
        ctx = StepContext(None, sum(q_lens), None, None, None, list(range(len(q_lens))), [int(s) for s in starts], q_lens,
                          [0] * len(q_lens), page_tokens=page_tokens)
        return part.step_tables(ctx).info.nw

    assert rows_per_item([2048]) == 16 and rows_per_item([1024]) == 16     # 256 and 128 items of 256 rows
    assert rows_per_item([512]) == 8 and rows_per_item([960]) == 8         # 64 and 120 items: one tile per CTA fills more SMs
    assert rows_per_item([512, 512]) == 16 and rows_per_item([700, 333]) == 16
    assert rows_per_item([2048], page_tokens=12) == 8                        # pages that are no 16 * 2^n tokens
    assert rows_per_item([1] * 8) == 1                                      # decode

"""The engine against the plain implementation, under every way of cutting the work.

For each tiny configuration and both precisions, the same requests are replayed whole, with
the last 32 tokens one by one, in portions of changing size, and mixed (up to four live
requests, portions beside decoded tokens, a pool so small that pages are used again); the
logits at every position are compared with the plain implementation's.  Tolerances were
fixed from the rounding model (float32: accumulated rounding of a few dozen operations;
bfloat16: inputs of every matrix product and the cache rounded to 8 bits of mantissa) and
are not to be widened.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen3

pytestmark = pytest.mark.gpu

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)

# max |difference| and mean |difference|, relative to the largest |logit| of the request set
TOL = {torch.float32: (2e-5, 2e-6), torch.bfloat16: (2e-2, 3e-3)}

CASES = {
    "A": dict(lengths=[7, 16, 33, 70], page_tokens=4),
    "B": dict(lengths=[5, 19, 64, 100], page_tokens=8),
    "C": dict(lengths=[40, 90, 130, 61, 77], page_tokens=16),
    "D": dict(lengths=[150, 37, 260, 90], page_tokens=16),
    "E": dict(lengths=[200, 75, 140], page_tokens=32),
    "F": dict(lengths=[3, 50, 121], page_tokens=16),
    "G": dict(lengths=[45, 8, 97], page_tokens=8),
}

_cache = {}


def setup_case(tmp_path_factory, which, dtype):
    key = (which, dtype)
    if key not in _cache:
        d = helpers.make_model_dir(tmp_path_factory.mktemp("models"), which, dtype)
        cfg, weights = helpers.load_plain(d)
        rng = np.random.default_rng(11)
        seqs = {f"r{i}": p for i, p in enumerate(helpers.prompts_for(which, rng, CASES[which]["lengths"]))}
        ref = {rid: plain_qwen3.forward(cfg, weights, ids) for rid, ids in seqs.items()}
        _cache[key] = (d, seqs, ref)
    return _cache[key]


def compare(got, ref, seqs, dtype):
    assert len(got) == sum(len(v) for v in seqs.values())
    scale = max(np.abs(r).max() for r in ref.values())
    tol_max, tol_mean = TOL[dtype]
    worst, where = 0.0, None
    means = []
    for (rid, p), v in sorted(got.items()):
        assert np.isfinite(v).all(), f"non-finite logits at {rid}:{p}"
        d = np.abs(v.astype(np.float64) - ref[rid][p])
        means.append(d.mean())
        if d.max() > worst:
            worst, where = d.max(), (rid, p)
    # report the FIRST position out of tolerance: its place says what is special about it
    for (rid, p), v in sorted(got.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        d = np.abs(v.astype(np.float64) - ref[rid][p]).max()
        assert d <= tol_max * scale, (
            f"first wrong position: request {rid} position {p}: |diff| {d:.3g} > {tol_max * scale:.3g} "
            f"(worst {worst:.3g} at {where})")
    assert np.mean(means) <= tol_mean * scale


def families(seqs):
    return {
        "whole": helpers.trace_whole(seqs),
        "tail": helpers.trace_tail_decode(seqs, 32),
        "portions": helpers.trace_portions(seqs),
        "mixed": helpers.trace_mixed(seqs, np.random.default_rng(3), max_live=4),
        "mixed_tight": helpers.trace_mixed(seqs, np.random.default_rng(4), max_live=2, prefill_chunks=(2, 9, 3, 21)),
    }


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E", "F", "G"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed", "mixed_tight"])
def test_replay_matches_plain(tmp_path_factory, which, dtype, family):
    from hk_b200.engine import Engine
    d, seqs, ref = setup_case(tmp_path_factory, which, dtype)
    steps = families(seqs)[family]
    max_tokens = helpers.peak_tokens(steps)
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=CASES[which]["page_tokens"],
                    max_requests=4, max_context=max_tokens)
    got = helpers.run_trace_on_engine(engine, steps)
    engine.cache.books.audit()
    assert all(f == engine.cache.num_pages for f in engine.free_pages()), "pages were not all given back"
    compare(got, ref, seqs, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which,page_tokens", [("D", 12), ("E", 12), ("B", 12), ("D", 1), ("A", 1), ("C", 1), ("G", 3)])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed", "mixed_tight"])
def test_replay_with_pages_that_are_no_power_of_two_and_pages_of_one_token(tmp_path_factory, which, page_tokens, dtype, family):
    """The engine takes any page size from one token up: a page of 12 tokens puts page edges where no 64-key tile and
    no 16-byte group ends, a page of one token makes every key a page of its own (the block table is as long as
    the context).  Same requests, same plain logits."""
    from hk_b200.engine import Engine
    d, seqs, ref = setup_case(tmp_path_factory, which, dtype)
    steps = families(seqs)[family]
    max_tokens = helpers.peak_tokens(steps, quantum=max(64, page_tokens))
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=page_tokens, max_requests=4, max_context=max_tokens)
    got = helpers.run_trace_on_engine(engine, steps)
    engine.cache.books.audit()
    assert all(f == engine.cache.num_pages for f in engine.free_pages()), "pages were not all given back"
    compare(got, ref, seqs, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which,page_tokens", [("D", 16), ("E", 32), ("B", 8)])
def test_replay_mixed_with_twelve_live_requests(tmp_path_factory, which, page_tokens, dtype):
    """Up to twelve live requests: steps that mix portions of several prompts with decoded tokens of many others,
    pure decode steps of 9 to 12 rows (captured graphs of 16 rows, filled up with repeats of the last row), pages
    that come back and are used again; every position against the plain implementation, in both precisions."""
    from hk_b200.engine import Engine
    d, _, _ = setup_case(tmp_path_factory, which, dtype)
    cfg, weights = helpers.load_plain(d)
    rng = np.random.default_rng(21)
    lengths = [int(n) for n in rng.integers(18, 90, 16)]
    seqs = {f"m{i}": p for i, p in enumerate(helpers.prompts_for(which, rng, lengths))}
    ref = {rid: plain_qwen3.forward(cfg, weights, ids) for rid, ids in seqs.items()}
    steps = helpers.trace_mixed(seqs, np.random.default_rng(5), max_live=12, prefill_chunks=(13, 5, 2, 29, 8), decode_tail=20)
    decode_rows = [len(st["entries"]) for st in steps if all(len(t) == 1 for _, t, _ in st["entries"])]
    assert max(len(st["entries"]) for st in steps) >= 10 and any(9 <= n <= 12 for n in decode_rows)
    max_tokens = helpers.peak_tokens(steps)
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=page_tokens, max_requests=12, max_context=128)
    got = helpers.run_trace_on_engine(engine, steps)
    engine.cache.books.audit()
    assert all(f == engine.cache.num_pages for f in engine.free_pages())
    if engine.decode_graphs:
        assert 16 in engine._graphs
    compare(got, ref, seqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path_factory, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON lines in, <step>.f32 files and `done` lines out."""
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, seqs, ref = setup_case(tmp_path_factory, "B", tdt)
    steps = families(seqs)["mixed"]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(helpers.peak_tokens(steps))],
        input=helpers.trace_to_jsonl(steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    vocab = helpers.TINY["B"][0]["vocab_size"]
    got, pos = {}, {}
    for i, st in enumerate(steps):
        wanted = sum(len(w) for _, _, w in st["entries"])
        path = out / f"{i}.f32"
        if wanted == 0:
            assert not path.exists()
        else:
            arr = np.fromfile(path, dtype="<f4").reshape(wanted, vocab)
            r = 0
            for rid, toks, want in st["entries"]:
                for w in want:
                    got[(rid, pos.get(rid, 0) + w)] = arr[r]
                    r += 1
        for rid, toks, _ in st["entries"]:
            pos[rid] = pos.get(rid, 0) + len(toks)
    compare(got, ref, seqs, tdt)

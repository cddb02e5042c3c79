"""Single-kernel cases with device timing: `python -m hk_b200.profiling <case> [sizes]`.

Each case sets up one hot kernel of the engine at a serving size, runs it a few times, times it
with CUDA events (L2 flushed between runs by reading a buffer larger than L2) and prints the
achieved GB/s or TFLOP/s.  The same command under `ncu -k regex:<kernel>` gives the hardware
counters for that kernel.  (The reference has per-kernel event timing of the same kind behind
HK_CUDA_EVENTS: src/cuda.zig:1212-1263.)

Cases: gemm_tc (tcgen05 product, --swiglu / --add), gemm_smallm and gemm_stream (decode products), attn_decode
(paged decode attention), attn_prefill (paged causal attention of one prompt), decode (whole decode steps
of a shallow random model with the 8B layer sizes, launched one kernel after the other without a graph: the
launch list of a profiler then shows every kernel of a step with its time).
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch


def _time(fn, reps: int, flush: torch.Tensor):
    times = []
    for i in range(reps + 2):
        if flush is not None:
            flush.max()       # reading a buffer larger than L2 leaves it full of clean lines that are not the case's
        else:
            torch.cuda._sleep(300000)     # L2 left as the run before left it; the GPU idles while the host launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(a.elapsed_time(b) * 1e3)
    return float(np.median(times))


def _paged(batch, ctx, G, hd, pt, dev):
    pages_per = -(-ctx // pt)
    n_pages = batch * pages_per
    k = torch.randn(n_pages, G, pt, hd, device=dev).to(torch.bfloat16)
    v = torch.randn(n_pages, G, pt, hd, device=dev).to(torch.bfloat16)
    perm = torch.randperm(n_pages, device=dev).to(torch.int32).view(batch, pages_per)
    return k, v, perm.contiguous()


def _decode_steps(a, dev) -> int:
    from .config import config_from_dict
    from .engine import Engine, StepEntry
    cfg = config_from_dict(dict(architectures=["Qwen3ForCausalLM"], hidden_size=a.hidden, num_hidden_layers=a.layers,
                                intermediate_size=a.intermediate, num_attention_heads=a.heads, num_key_value_heads=a.kv_heads,
                                head_dim=a.head_dim, vocab_size=a.vocab, rope_theta=1e6, rms_norm_eps=1e-6,
                                tie_word_embeddings=False, max_position_embeddings=8192, initializer_range=0.02))
    per = -(-(a.ctx + 64) // 64) * 64
    eng = Engine(config=cfg, random_seed=2, dtype="bfloat16", max_tokens=a.batch * per, page_tokens=a.page_tokens,
                 max_requests=a.batch, max_context=8192, max_batch_tokens=8192, decode_graphs=False)
    rng = np.random.default_rng(0)
    ids = list(range(a.batch))
    for r in ids:
        eng.open_request(r)
    group = max(1, 8192 // a.ctx)
    for i in range(0, a.batch, group):
        eng.step([StepEntry(r, rng.integers(0, a.vocab, a.ctx).tolist(), []) for r in ids[i:i + group]])
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for s in range(a.reps):
        if s == a.reps - 1:
            t0.record()
        eng.step([StepEntry(r, [int(rng.integers(0, a.vocab))], [0]) for r in ids])
    t1.record()
    torch.cuda.synchronize()
    print(f"decode layers={a.layers} batch={a.batch} ctx={a.ctx}: last step {t0.elapsed_time(t1) * 1e3:.0f} us (no graph)")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hk_b200.profiling")
    ap.add_argument("case", choices=["gemm_tc", "gemm_smallm", "gemm_stream", "attn_decode", "attn_prefill", "decode"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--add", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page-tokens", type=int, default=16)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--splits", type=int, default=0, help="attn_decode: key splits per request and kv head (default: as the decode graphs choose); gemm_tc: K slices")
    ap.add_argument("--bn", type=int, default=0, help="gemm_tc: pin the tile width (a multiple of 16, of 32 with --swiglu, up to 256)")
    ap.add_argument("--warm", action="store_true", help="do not flush L2 between the timed runs")
    ap.add_argument("--layers", type=int, default=2, help="decode: layers of the model")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--mma", action="store_true", help="attn_prefill: the mma.sync kernel instead of the tcgen05 one")
    ap.add_argument("--one-tile", action="store_true", help="attn_prefill: the tcgen05 kernel with one query tile per CTA")
    ap.add_argument("--row-warps", type=int, default=0, help="gemm_stream: consumer warps across a tile's rows (8, 4, 2 or 1)")
    ap.add_argument("--ctas", type=int, default=0, help="gemm_stream: run this many CTAs instead of one per SM")
    ap.add_argument("--row-tiles", type=int, default=0, help="gemm_smallm: pin the row tiles of 16 per CTA (1, 2 or 4)")
    a = ap.parse_args(argv)
    from .csrc import attention_fast, gemm_fast, ops
    gemm_fast._rt_override = a.row_tiles
    gemm_fast._stream_ctas = a.ctas
    if a.case == "gemm_tc":
        gemm_fast._tc_bn, gemm_fast._tc_splits = a.bn, a.splits
    if a.row_warps:
        gemm_fast._stream_rw = a.row_warps
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = None if a.warm else torch.zeros(64 << 20, dtype=torch.int32, device=dev)      # larger than the 126 MB L2
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    if a.case == "decode":
        return _decode_steps(a, dev)
    if a.case in ("gemm_tc", "gemm_smallm", "gemm_stream"):
        x = (torch.randn(a.m, a.k, device=dev) / 8).to(torch.bfloat16)
        w = (torch.randn(a.n, a.k, device=dev) / 8).to(torch.bfloat16)
        if a.swiglu:
            out = torch.empty(a.m, a.n // 2, dtype=torch.bfloat16, device=dev)
            fn = lambda: ops.gemm_swiglu(x, w, out)
        else:
            out = torch.zeros(a.m, a.n, dtype=torch.float32, device=dev)
            fn = lambda: ops.gemm(x, w, out, accumulate=a.add)
        with ops.force(gemm={"gemm_tc": "tc", "gemm_smallm": "smallm", "gemm_stream": "stream"}[a.case]):
            us = _time(fn, a.reps, flush)
        flops = 2.0 * a.m * a.n * a.k
        nbytes = 2.0 * (a.n * a.k + a.m * a.k) + out.numel() * out.element_size()
        print(f"{a.case} M={a.m} N={a.n} K={a.k} swiglu={a.swiglu} add={a.add}: {us:.1f} us, "
              f"{flops / us * 1e-6:.1f} TFLOP/s, {nbytes / us * 1e-3:.1f} GB/s")
    else:
        H, G, hd, pt = a.heads, a.kv_heads, a.head_dim, a.page_tokens
        scale = 1.0 / math.sqrt(hd)
        upload = lambda arr: torch.from_numpy(np.ascontiguousarray(arr)).to(dev)
        if a.case == "attn_decode":
            k, v, bt = _paged(a.batch, a.ctx, G, hd, pt, dev)
            n = a.batch
            q = torch.randn(n, H * hd, device=dev).to(torch.bfloat16)
            pos = torch.full((n,), a.ctx - 1, dtype=torch.int32, device=dev)
            slot = torch.arange(n, dtype=torch.int32, device=dev)
            splits = a.splits or attention_fast.decode_splits(n, G, sms)
            plan = attention_fast.build_plan(list(range(n)), list(range(n)), [1] * n, [a.ctx - 1] * n, n, 0, H, G, sms, upload,
                                             fixed_splits=splits)
            nbytes = 2.0 * 2 * n * a.ctx * G * hd
            flops = 4.0 * n * H * hd * a.ctx
        else:
            k, v, bt = _paged(1, a.ctx, G, hd, pt, dev)
            n = a.ctx
            q = torch.randn(n, H * hd, device=dev).to(torch.bfloat16)
            pos = torch.arange(n, dtype=torch.int32, device=dev)
            slot = torch.zeros(n, dtype=torch.int32, device=dev)
            rows = 64
            if attention_fast.tc_prefill_supported(hd, H // G) and not a.mma:
                rows = 256 if attention_fast.tc2_prefill_supported(hd, H // G, pt) and not a.one_tile else 128
            plan = attention_fast.build_plan([0], [0], [n], [0], n, 0, H, G, sms, upload, prefill_rows=rows)
            nbytes = 2.0 * 2 * n * G * hd + 2 * 2.0 * n * H * hd
            flops = 4.0 * H * hd * n * (n + 1) / 2
        out = torch.empty_like(q)
        fn = lambda: ops.paged_attention(q, k, v, bt, pos, slot, out, H, G, hd, pt, 0, scale, plan=plan)
        us = _time(fn, a.reps, flush)
        print(f"{a.case} batch={a.batch} ctx={a.ctx} H={H} G={G} hd={hd} page={pt}: {us:.1f} us, "
              f"{flops / us * 1e-6:.1f} TFLOP/s, {nbytes / us * 1e-3:.1f} GB/s (cache bytes / time)")
    gemm_fast.check_status(dev)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

#!/usr/bin/env python3
"""Serving benchmark of the engine on one B200: Qwen3-8B shape, random weights, bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 over a cache of 16-token pages
(a "step" is one decode step of the whole batch: forward over the paged cache, output head, greedy
pick), timed on the device with CUDA events after W warm-up steps; every request holds a 2,048-token
context when the timed steps begin.  A timed region is exactly K steps; it is repeated (`regions` in
`config`) and the median region is reported, with the range in `ms_per_step_range`.  `points` holds the
same at batch 1 and 64, and at all three batch sizes over 64-token pages (`*_page64`).  `roofline`
relates the batch-8 step's necessary bytes (every weight once, the cache of the live requests) to the
measured copy bandwidth; `roofline_points` does so for every batch size.  `e2e` is batch 8 through the
Python entry point (`generate_with_engine`: scheduler, host token ids in through pinned memory,
sampled ids back to the host every step); `e2e_points` the same at batch 1 and 64.  `prefill` is one
2,048-token prompt in one step (median of `--prefill-reps` runs), with its fraction of the measured
bf16 peak as a burst (`frac`) and sustained (`frac_sustained`).  Each timed step reads about 15 GB of
weights, far more than the 126 MB L2, so no flush is needed between steps (`l2` in `config` says so).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark configuration: the Qwen3-8B shape
SHAPE = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_hidden_layers=36, intermediate_size=12288,
             num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1000000.0,
             rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=8192, initializer_range=0.02)
CONTEXT = 8192
PROMPT = 2048
PAGE = 16             # the cache geometry of the benchmark configuration
PAGE_EXTRA = 64       # measured as extra points
REGIONS = 5           # timed regions of K steps each; the median is reported
SEED = 2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    try:
        with open(path) as f:
            m = json.load(f)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if isinstance(m.get(k), (int, float)) and m[k] > 0:
                out[k] = float(m[k])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, window=None):
        """Ends the sampling; the summary counts the samples taken inside `window` = (start, end) in time.time()
        seconds (the sampler is started earlier: nvidia-smi takes a moment to print its first line)."""
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz, mx, reasons = [], 0, set()
        for t, s in self.samples:
            if window is not None and not window[0] <= t <= window[1]:
                continue
            try:
                mhz.append(int(s[0]))
                mx = max(mx, int(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


def layer_param_count(c):
    d, F = c["hidden_size"], c["intermediate_size"]
    qd, kd = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    return d * (qd + 2 * kd) + qd * d + 3 * d * F


def decode_bytes(c, layers, batch, ctx_tokens):
    """Bytes one decode step has to read: every weight it uses once (bf16) and the cache of the live requests."""
    w = 2 * (layers * layer_param_count(c) + c["vocab_size"] * c["hidden_size"])
    kv = 2 * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * ctx_tokens * batch
    return w + kv


def prefill_flops(c, layers, t):
    gemm = 2 * t * (layers * layer_param_count(c) + c["vocab_size"] * c["hidden_size"] / t)
    attn = layers * 4 * c["num_attention_heads"] * c["head_dim"] * t * (t + 1) / 2
    return gemm + attn


def run(args):
    import numpy as np
    import torch

    import hk_b200
    from hk_b200.api import GenerationStats, generate_with_engine
    from hk_b200.config import config_from_dict
    from hk_b200.csrc import ops
    from hk_b200.engine import Engine, StepEntry

    shape = dict(SHAPE)
    layers_full = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    layers = shape["num_hidden_layers"]
    cfg = config_from_dict(shape)
    pk = peaks()
    batches = sorted({1, 8, 64} if not args.quick else {1, 8})
    regions = 1 if args.quick else REGIONS
    per_req = -(-(PROMPT + args.warmup + regions * args.steps + 8) // 64) * 64
    rng = np.random.default_rng(SEED)
    vocab = shape["vocab_size"]

    def make_engine(page, batch):
        """An engine sized for `batch` requests (slots and pages), as a server started for that load would be."""
        t_load = time.time()
        eng = Engine(config=cfg, random_seed=SEED, dtype="bfloat16", max_tokens=batch * per_req, page_tokens=page,
                     max_requests=batch, max_context=CONTEXT, max_batch_tokens=max(PROMPT, batch))
        torch.cuda.synchronize()
        print(f"[bench] model ready in {time.time() - t_load:.1f} s ({layers} of {layers_full} layers, {page}-token pages, "
              f"{batch} requests, {torch.cuda.memory_allocated() / 2**30:.1f} GiB on the device)", file=sys.stderr, flush=True)
        return eng

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill of 2,048 tokens (one step), timed on the device ----
    def prefill_point(engine):
        prompt = rng.integers(0, vocab, PROMPT).tolist()
        times = []
        for i in range(args.prefill_reps + 2):
            engine.open_request("p")
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            engine.step([StepEntry("p", prompt, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            engine.close_request("p")
            if i > 1:
                times.append(a.elapsed_time(b))
        ms = float(np.median(times))
        flops = prefill_flops(shape, layers, PROMPT)
        return {"value": PROMPT / ms * 1e3, "tokens": PROMPT, "ms": ms, "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12),
                "frac_sustained": flops / (ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12),
                "ms_range": [float(min(times)), float(max(times))], "reps": len(times)}

    # ---- decode at batch B: every request holds PROMPT tokens, then W warm-up steps and `regions` regions of K steps ----
    def decode_point(engine, batch, clocks=None):
        steps, warmup = args.steps, args.warmup
        ids = [f"d{i}" for i in range(batch)]
        for r in ids:
            engine.open_request(r)
        # fill the contexts: real prefill steps, several requests per step
        group = max(1, engine.max_batch_tokens // PROMPT)
        for i in range(0, batch, group):
            engine.step([StepEntry(r, rng.integers(0, vocab, PROMPT).tolist(), []) for r in ids[i:i + group]])
        toks = rng.integers(0, vocab, (warmup + regions * steps, batch))
        out = torch.empty(batch, dtype=torch.int32, device=engine.device)

        def one(s):
            logits = engine.step([StepEntry(r, [int(toks[s, i])], [0]) for i, r in enumerate(ids)])
            ops.argmax(logits, out)

        for s in range(warmup):
            one(s)
        if clocks is not None:
            clocks.start()
            time.sleep(0.3)             # nvidia-smi takes a moment to print its first line
        ms, launches, window = [], 0, [0.0, 0.0]
        for reg in range(regions):
            a, b = ev(), ev()
            torch.cuda.synchronize()
            if reg == 0:
                window[0] = time.time()
            l0 = ops.launch_count()
            a.record()
            for s in range(warmup + reg * steps, warmup + (reg + 1) * steps):
                one(s)
            b.record()
            torch.cuda.synchronize()
            window[1] = time.time()
            ms.append(a.elapsed_time(b) / steps)
            launches = ops.launch_count() - l0
        engine.check_kernel_status()
        for r in ids:
            engine.close_request(r)
        ctx_mid = PROMPT + warmup + regions * steps // 2
        nbytes = decode_bytes(shape, layers, batch, ctx_mid)
        med = float(np.median(ms))
        achieved = nbytes / (med * 1e-3) / 1e9
        return {"ms": med, "ms_range": [float(min(ms)), float(max(ms))], "launches": launches, "window": tuple(window),
                "tok_s": batch / med * 1e3,
                "roofline": {"bytes": nbytes, "ms": med, "achieved": achieved, "frac": achieved / pk["hbm_gbs"]}}

    # ---- end to end through the Python entry point ----
    def e2e_point(engine, batch):
        prompts = [rng.integers(0, vocab, PROMPT).tolist() for _ in range(batch)]
        st = GenerationStats()
        # as many new tokens as the decode point ran steps (its warm-up included): a tail of a few steps would mostly
        # time the hand-over from the last prompt portion to decoding
        generate_with_engine(engine, prompts, max_new_tokens=args.warmup + regions * args.steps + 1, temperature=0, top_k=0,
                             eos_token_ids=(), prefill_chunk=PROMPT, stats=st)
        return {"value": st.decode_tokens / max(st.decode_seconds, 1e-9), "unit": "tokens/s",
                "h2d_bytes_per_step": st.h2d_bytes_per_step, "d2h_bytes_per_step": st.d2h_bytes_per_step}

    import gc

    def drop():
        gc.collect()                    # an engine and its captured graphs refer to each other
        torch.cuda.empty_cache()

    dec, e2e = {}, {}
    pre = clock_info = None
    for bsz in [8] + [b for b in batches if b != 8]:          # the headline first
        engine = make_engine(PAGE, bsz)
        if bsz == 8:
            pre = prefill_point(engine)
            clocks = ClockSampler()
            dec[8] = decode_point(engine, 8, clocks)
            clock_info = clocks.stop(dec[8]["window"])
        else:
            dec[bsz] = decode_point(engine, bsz)
        e2e[bsz] = e2e_point(engine, bsz)
        e2e[bsz]["of_device_timed"] = e2e[bsz]["value"] / dec[bsz]["tok_s"]
        engine = None
        drop()
    points = {f"decode_b{b}": dec[b]["tok_s"] for b in batches if b != 8}
    roof_points = {f"decode_b{b}": dec[b]["roofline"] for b in batches}
    e2e_points = {f"decode_b{b}": e2e[b] for b in batches if b != 8}
    if not args.quick:
        # the same decode points over 64-token pages
        for bsz in batches:
            engine = make_engine(PAGE_EXTRA, bsz)
            d = decode_point(engine, bsz)
            points[f"decode_b{bsz}_page{PAGE_EXTRA}"] = d["tok_s"]
            roof_points[f"decode_b{bsz}_page{PAGE_EXTRA}"] = d["roofline"]
            engine = None
            drop()

    main = dec[8]
    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, 2,048-token contexts)",
        "value": main["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main["ms"], "ms_per_step_range": main["ms_range"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded uniform token ids, random-init weights N(0, 0.02) seed 2",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": layers_full, "hidden": shape["hidden_size"],
                   "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": vocab,
                   "global_batch": 8, "seq_len": PROMPT, "context": CONTEXT, "page_tokens": PAGE,
                   "page_tokens_extra_points": PAGE_EXTRA, "regions": regions, "engine": "one per batch size, sized for it",
                   "parallelism": "1 gpu", "l2": "each step reads >15 GB of weights, larger than L2; no flush",
                   "peaks": pk["source"]},
        "prefill": pre,
        "roofline": {"bound": "hbm", "achieved": main["roofline"]["achieved"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": main["roofline"]["frac"]},
        "roofline_points": roof_points,
        "points": points,
        "e2e": e2e[8],
        "e2e_points": e2e_points,
        "gpu_launches": main["launches"],
        "clocks": clock_info,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (named in `config`)")
    ap.add_argument("--prefill-reps", type=int, default=7)
    ap.add_argument("--quick", action="store_true", help="skip batch 64")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Zig project (build.zig); no Zig toolchain is installed and none can be fetched, "
                          "so its engine cannot be built here; its Python package alone has no Qwen3 engine without the native library"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path (asked for --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    run(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())

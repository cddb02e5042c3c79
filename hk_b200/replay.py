"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives `Engine`,
the one that generation uses.  The reference's analogue is `hk-probe` (ids in, raw
little-endian float32 logits out: tools/hk_probe.zig:100-124; `--multi` steps several
sequences together: :263-315).

Input, one JSON object a line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: for each request its next tokens and the places among them whose logits are
wanted; all entries of a step run as one batch.  `end`: requests finished after this step;
their pages and slot are given back.  For a step in which something is wanted,
`<out>/<step>.f32` receives the logits [wanted, vocab] as little-endian float32, in the
order of the entries and of `want`.  After every step a line `done <step>` is printed and
flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--page-tokens", type=int, default=16)
    args = ap.parse_args(argv)
    if args.max_tokens < 1:
        ap.error("--max-tokens must be positive")

    from .engine import Engine, StepEntry
    os.makedirs(args.out, exist_ok=True)
    print(f"[trace_run] loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    engine = Engine(args.model, dtype=args.dtype, max_tokens=args.max_tokens, page_tokens=args.page_tokens,
                    max_requests=args.max_requests, max_context=args.max_tokens,
                    max_batch_tokens=args.max_tokens)
    import numpy as np
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not engine.has_request(rid):
                engine.open_request(rid)
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            engine.check_kernel_status()          # no logits leave with a kernel's time-out unreported
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            engine.close_request(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())

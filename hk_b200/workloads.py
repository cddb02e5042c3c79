"""Serving workloads through the scheduler at the layer sizes of the larger models of the family:
`python -m hk_b200.workloads <name> [--layers N]`.

The engine's throughput figures come from steps of one kind (a prompt alone, a batch of decoded tokens).  These
two workloads run what a server sees: many requests of different lengths, prompts cut into portions and fed beside
the decoded tokens of the requests that are further on, sampling with temperature, requests that finish at different
times.  Random weights, seeded uniform token ids; one line of JSON on standard output.

* `serve14b`: hidden 5120, 40 query and 8 key heads of 128, feed-forward 17,408, 40 layers.  32 requests with
  prompt lengths uniform in [128, 4096], all submitted at once, portions of 512 tokens beside decoding, 128 new
  tokens each at temperature 0.8.
* `mixed32b`: hidden 5120, 64 query and 8 key heads of 128, feed-forward 25,600, 64 layers.  8 requests decoding at
  a context of 6,000 tokens when 8 prompts of 1,024 tokens arrive; greedy, 64 new tokens each.  The clock starts when
  the new prompts arrive.

(The reference's own benchmark drives its engine with synthetic ids of given lengths in the same way:
tools/hk_probe.zig:184,263-315.)
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np
import torch

SHAPES = {
    "serve14b": dict(hidden_size=5120, num_hidden_layers=40, intermediate_size=17408, num_attention_heads=40,
                     num_key_value_heads=8, head_dim=128, vocab_size=151936),
    "mixed32b": dict(hidden_size=5120, num_hidden_layers=64, intermediate_size=25600, num_attention_heads=64,
                     num_key_value_heads=8, head_dim=128, vocab_size=151936),
}
PAGE = 64


def _opt(args, name, default):
    """An override of a workload's constants (tests run the workloads small, greedy and in either precision)."""
    v = getattr(args, name, None)
    return default if v is None else v


def _engine(name: str, layers: int, seed: int, lengths, max_batch_tokens: int, dtype: str = "bfloat16"):
    from .config import config_from_dict
    from .engine import Engine
    shape = dict(SHAPES[name])
    if layers:
        shape["num_hidden_layers"] = layers
    cfg = config_from_dict(dict(architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                max_position_embeddings=8192, initializer_range=0.02, **shape))
    tokens = sum(-(-n // PAGE) * PAGE for n in lengths)
    eng = Engine(config=cfg, random_seed=seed, dtype=dtype, max_tokens=tokens, page_tokens=PAGE, max_requests=len(lengths),
                 max_context=8192, max_batch_tokens=max_batch_tokens)
    return cfg, eng


def _drain(sched, counters):
    """Steps the scheduler until nothing is left; counts the steps that carried prompt portions beside decoded tokens."""
    while sched.has_work():
        p0, d0 = sched.stats.prompt_tokens, sched.stats.decode_tokens
        sched.step()
        if sched.stats.prompt_tokens != p0 and sched.stats.decode_tokens != d0:
            counters["mixed_steps"] += 1


def serve14b(args) -> dict:
    from .engine.scheduler import Scheduler
    from .sampling import SamplingParams
    rng = np.random.default_rng(3)
    n_req, new = 32, _opt(args, "new_tokens", 128)
    lo, hi = _opt(args, "prompt_range", (128, 4096))
    temperature = _opt(args, "temperature", 0.8)
    lens = rng.integers(lo, hi + 1, n_req).tolist()
    cfg, eng = _engine("serve14b", args.layers, 3, [n + new for n in lens], max_batch_tokens=2048, dtype=_opt(args, "dtype", "bfloat16"))
    prompts = [rng.integers(0, cfg.vocab_size, n).tolist() for n in lens]

    def once():
        sched = Scheduler(eng, prefill_chunk=_opt(args, "portion", 512))
        ids = [sched.submit(p, new, SamplingParams(temperature=temperature, top_k=0, top_p=1.0, min_p=0.0, seed=100 + i))
               for i, p in enumerate(prompts)]
        counters = {"mixed_steps": 0}
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _drain(sched, counters)
        torch.cuda.synchronize()
        if _opt(args, "keep_tokens", False):
            args.kept = (cfg, prompts, [list(sched.finished[i].output) for i in ids])
        return sched, counters, time.perf_counter() - t0, sum(len(sched.finished[i].output) for i in ids)

    first = once()[2]            # loads the kernels and captures the decode graphs of every batch size it meets
    sched, counters, dt, out = once()
    eng.cache.books.audit()
    return {"workload": "serve14b", "layers": cfg.num_hidden_layers, "layers_full": SHAPES["serve14b"]["num_hidden_layers"],
            "requests": n_req, "prompt_tokens": int(sum(lens)), "generated_tokens": out, "seconds": dt, "first_run_seconds": first,
            "tokens_per_s": (sum(lens) + out) / dt, "generated_per_s": out / dt, "steps": sched.stats.steps,
            "mixed_steps": counters["mixed_steps"], "ahead_steps": sched.stats.ahead_steps, "preemptions": sched.stats.preemptions,
            "portion": _opt(args, "portion", 512), "temperature": temperature, "page_tokens": PAGE,
            "dtype": _opt(args, "dtype", "bfloat16"), "data": "synthetic ids, random weights"}


def mixed32b(args) -> dict:
    from .engine.scheduler import Scheduler
    from .sampling import SamplingParams
    rng = np.random.default_rng(4)
    ctx, new_len, new = _opt(args, "context", 6000), _opt(args, "new_prompt", 1024), _opt(args, "new_tokens", 64)
    # the old requests decode one token while the prompts are fed and 64 more beside the new requests
    lengths = [ctx + 2 * new + 8] * 8 + [new_len + new] * 8
    cfg, eng = _engine("mixed32b", args.layers, 4, lengths, max_batch_tokens=4096, dtype=_opt(args, "dtype", "bfloat16"))
    greedy = SamplingParams(temperature=0.0)
    sched = Scheduler(eng, prefill_chunk=_opt(args, "portion", 1024))
    old_prompts = [rng.integers(0, cfg.vocab_size, ctx - 1).tolist() for _ in range(8)]
    old = [sched.submit(p, new + 1, greedy) for p in old_prompts]
    while len(sched.running) < 8 or not all(r.output for r in sched.running):
        sched.step()                                       # the old requests' prompts, then their first token
    torch.cuda.synchronize()
    counters = {"mixed_steps": 0}
    fresh_prompts = [rng.integers(0, cfg.vocab_size, new_len).tolist() for _ in range(8)]
    fresh = [sched.submit(p, new, greedy) for p in fresh_prompts]
    steps0, dec0 = sched.stats.steps, sum(len(r.output) for r in sched.running)
    t0 = time.perf_counter()
    _drain(sched, counters)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    out = sum(len(sched.finished[i].output) for i in old + fresh) - dec0
    eng.cache.books.audit()
    if _opt(args, "keep_tokens", False):
        args.kept = (cfg, old_prompts + fresh_prompts, [list(sched.finished[i].output) for i in old + fresh])
    return {"workload": "mixed32b", "layers": cfg.num_hidden_layers, "layers_full": SHAPES["mixed32b"]["num_hidden_layers"],
            "requests": 16, "decoding_context": ctx, "new_prompt_tokens": 8 * new_len, "generated_tokens": out, "seconds": dt,
            "tokens_per_s": (8 * new_len + out) / dt, "generated_per_s": out / dt, "steps": sched.stats.steps - steps0,
            "mixed_steps": counters["mixed_steps"], "ahead_steps": sched.stats.ahead_steps, "preemptions": sched.stats.preemptions,
            "page_tokens": PAGE, "dtype": _opt(args, "dtype", "bfloat16"), "data": "synthetic ids, random weights"}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("workload", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (named in the output)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print("hk_b200.workloads needs a GPU", file=sys.stderr)
        return 1
    print(json.dumps({"serve14b": serve14b, "mixed32b": mixed32b}[args.workload](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""`hk run`: the command line, with the reference's option names and meanings
(tools/hk_cli.zig:1717-1738 usage, :1819-1859 parsing).

Differences that the scope forces: the model is a folder with config.json and safetensors
(not a .hk file), and the prompt is a list of token ids ("12,7,99" or "12 7 99") because
tokenizers are outside this engine; generated ids go to standard output, the statistics
line to standard error (as :1599-1602,1702-1715).  An unknown or malformed flag is an error
before the model is touched (:1817-1859).  `--threads`, `-ngl/--gpu-layers` and `--backend`
are accepted for compatibility: this engine always runs whole on one CUDA device.
"""
from __future__ import annotations

import sys
import time

USAGE = """Usage: hk run <model folder> [token ids | -p IDS] [options]

  -p, --prompt IDS      token ids to continue, separated by commas or spaces (a bare argument works too)
  -n, --max-tokens N    most tokens to generate (default 128)
      --temp T          temperature, 0 picks the most likely token (default 0.8)
      --top-k N         keep the N most likely tokens, 0 for no limit (default 40)
      --top-p P         nucleus sampling, 1 to disable (default 0.95)
      --min-p P         drop tokens below P times the best one (default 0.05)
      --repeat-penalty X  penalty for recent tokens, 1 to disable (default 1.0)
      --seed N          random seed, 0 uses the clock (default 0)
      --threads N       accepted, unused: the work runs on the GPU
  -ngl, --gpu-layers N  accepted: the whole model always runs on the GPU; 0 is refused (no CPU path)
      --backend B       auto | cuda; cpu and vulkan are refused (this engine is CUDA only)
      --dtype D         bfloat16 | float32 (default bfloat16)
      --max-ctx N       context length to provide (default: prompt + max tokens, rounded up to 64)
      --prompt-len N    instead of a prompt: N token ids drawn uniformly from the vocabulary with --seed
      --page-tokens N   tokens per cache page (default 64)

       hk random <config.json> <new model folder> [--seed N] [--dtype D] [--std S]
                        writes config.json and model.safetensors with seeded random weights
"""


class BadUsage(Exception):
    pass


def _fail(msg: str):
    raise BadUsage(msg)


def _need_value(args, i, flag):
    if i + 1 >= len(args):
        _fail(f"Error: '{flag}' needs a value")
    return args[i + 1]


def _uint(args, i, flag, minimum):
    v = _need_value(args, i, flag)
    try:
        n = int(v)
    except ValueError:
        _fail(f"Error: '{flag}' got '{v}', expected a whole number")
    if n < minimum:
        _fail(f"Error: '{flag}' got '{v}', expected at least {minimum}")
    return n


def _float_in(args, i, flag, lo, hi, what):
    v = _need_value(args, i, flag)
    try:
        x = float(v)
    except ValueError:
        _fail(f"Error: '{flag}' got '{v}', expected {what}")
    if not lo <= x <= hi:
        _fail(f"Error: '{flag}' got '{v}', expected {what}")
    return x


def parse_ids(text: str):
    parts = text.replace(",", " ").split()
    if not parts:
        _fail("Error: the prompt produced no tokens.")
    try:
        ids = [int(p) for p in parts]
    except ValueError:
        _fail(f"Error: the prompt '{text}' is not a list of token ids")
    if any(t < 0 for t in ids):
        _fail("Error: token ids cannot be negative")
    return ids


def parse_run_args(args):
    """Returns a dict of settings; raises BadUsage on anything unknown or malformed."""
    g = dict(model=None, prompt=None, max_tokens=128, temperature=0.8, top_k=40, top_p=0.95, min_p=0.05,
             repeat_penalty=1.0, seed=0, dtype="bfloat16", max_ctx=None, prompt_len=None, page_tokens=None)
    i = 0
    while i < len(args):
        flag = args[i]
        if flag in ("-p", "--prompt"):
            if g["prompt"] is not None:
                _fail("Error: more than one prompt was given. Quote the prompt so it is one argument.")
            g["prompt"] = _need_value(args, i, flag)
            i += 2
        elif flag in ("-n", "--max-tokens"):
            g["max_tokens"] = _uint(args, i, flag, 1)
            i += 2
        elif flag in ("-ngl", "--gpu-layers"):
            if _uint(args, i, flag, 0) == 0:
                _fail("Error: '-ngl 0' asks for the CPU; this engine has no CPU path")
            i += 2
        elif flag == "--backend":
            v = _need_value(args, i, flag)
            if v not in ("auto", "cpu", "vulkan", "cuda"):
                _fail(f"Error: '--backend' got '{v}', expected auto, cpu, vulkan or cuda")
            if v in ("cpu", "vulkan"):
                _fail(f"Error: backend '{v}' is not part of this engine (CUDA only)")
            i += 2
        elif flag == "--threads":
            _uint(args, i, flag, 1)
            i += 2
        elif flag == "--temp":
            g["temperature"] = _float_in(args, i, flag, 0, 100, "a number from 0 up")
            i += 2
        elif flag == "--top-k":
            g["top_k"] = _uint(args, i, flag, 0)
            i += 2
        elif flag == "--top-p":
            g["top_p"] = _float_in(args, i, flag, 0, 1, "a number from 0 to 1")
            i += 2
        elif flag == "--min-p":
            g["min_p"] = _float_in(args, i, flag, 0, 1, "a number from 0 to 1")
            i += 2
        elif flag in ("--repeat-penalty", "--rep-pen"):
            g["repeat_penalty"] = _float_in(args, i, flag, 0.01, 100, "a positive number")
            i += 2
        elif flag == "--seed":
            g["seed"] = _uint(args, i, flag, 0)
            i += 2
        elif flag == "--dtype":
            v = _need_value(args, i, flag)
            if v not in ("bfloat16", "float32"):
                _fail(f"Error: '--dtype' got '{v}', expected bfloat16 or float32")
            g["dtype"] = v
            i += 2
        elif flag == "--max-ctx":
            g["max_ctx"] = _uint(args, i, flag, 1)
            i += 2
        elif flag == "--prompt-len":
            g["prompt_len"] = _uint(args, i, flag, 1)
            i += 2
        elif flag == "--page-tokens":
            g["page_tokens"] = _uint(args, i, flag, 1)
            i += 2
        elif flag.startswith("-") and len(flag) > 1 and not flag[1:].replace(",", "").replace(" ", "").isdigit():
            _fail(f"Error: unknown argument '{flag}'")
        elif g["model"] is None:
            g["model"] = flag
            i += 1
        else:
            if g["prompt"] is not None:
                _fail("Error: more than one prompt was given. Quote the prompt so it is one argument.")
            g["prompt"] = flag
            i += 1
    if g["model"] is None:
        _fail("Error: no model folder was given")
    if g["prompt"] is not None and g["prompt_len"] is not None:
        _fail("Error: both a prompt and '--prompt-len' were given")
    if g["prompt"] is None and g["prompt_len"] is None:
        _fail("Error: no prompt. Give one as a bare argument or with -p.")
    g["prompt_ids"] = parse_ids(g["prompt"]) if g["prompt"] is not None else None     # None: drawn once the vocabulary is known
    return g


def cmd_run(args) -> int:
    try:
        g = parse_run_args(args)
    except BadUsage as e:
        print(f"{e}\n{USAGE}", file=sys.stderr, end="")
        return 2
    from .api import GenerationStats, generate_with_engine
    from .config import ConfigError
    from .engine import Engine, EngineError
    from .weights import SafetensorsError, WeightError
    ids = g["prompt_ids"]
    n_prompt = len(ids) if ids is not None else g["prompt_len"]
    ctx = g["max_ctx"] or -(-(n_prompt + g["max_tokens"]) // 64) * 64
    try:
        t0 = time.perf_counter()
        from .api import SERVING_PAGE_TOKENS
        engine = Engine(g["model"], dtype=g["dtype"], max_tokens=ctx, page_tokens=g["page_tokens"] or SERVING_PAGE_TOKENS,
                        max_requests=1, max_context=ctx, max_batch_tokens=max(ctx, 1))
        if ids is None:
            import numpy as np
            ids = np.random.default_rng(g["seed"]).integers(0, engine.vocab, n_prompt).tolist()
        if any(t >= engine.vocab for t in ids):
            print(f"Error: a token id is outside the vocabulary of {engine.vocab}", file=sys.stderr)
            return 1
        load_s = time.perf_counter() - t0
        # prompt and generation are timed apart, as the reference's statistics line does
        import torch
        from .engine.scheduler import Scheduler
        from .sampling import SamplingParams
        # one request, nobody waits behind its prompt: portions of 2,048 tokens, where the prefill kernels run best
        sched = Scheduler(engine, prefill_chunk=2048, eos_token_ids=getattr(engine.config, "eos_token_ids", ()))
        rid = sched.submit(ids, g["max_tokens"], SamplingParams(
            temperature=g["temperature"], top_k=g["top_k"], top_p=g["top_p"], min_p=g["min_p"],
            repeat_penalty=g["repeat_penalty"], seed=g["seed"]))
        t1 = time.perf_counter()
        first = True
        prompt_s = 0.0
        printed = 0
        while sched.has_work():
            sched.step()
            req = (sched.finished.get(rid) or next(r for r in sched.running + list(sched.queue) if r.id == rid))
            if first and req.output:
                torch.cuda.synchronize()
                prompt_s = time.perf_counter() - t1
                first = False
            for tok in req.output[printed:]:
                sys.stdout.write(("" if printed == 0 else " ") + str(tok))
                printed += 1
            sys.stdout.flush()
        torch.cuda.synchronize()
        gen_s = time.perf_counter() - t1 - prompt_s
        produced = len(sched.finished[rid].output)
        mem = torch.cuda.max_memory_allocated() / (1 << 20)
        print(f"\n\n[prompt {len(ids)} tok (0 cached), {len(ids) / max(prompt_s, 1e-9):.1f} tok/s | "
              f"generated {produced} tok, {max(produced - 1, 0) / max(gen_s, 1e-9):.1f} tok/s | "
              f"memory {mem:.0f} MiB on the GPU | load {load_s:.1f} s]", file=sys.stderr)
        return 0
    except (ConfigError, WeightError, SafetensorsError, EngineError, FileNotFoundError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1


def parse_random_args(args):
    g = dict(config=None, out=None, seed=0, dtype="bfloat16", std=None)
    i = 0
    while i < len(args):
        flag = args[i]
        if flag == "--seed":
            g["seed"] = _uint(args, i, flag, 0)
            i += 2
        elif flag == "--dtype":
            v = _need_value(args, i, flag)
            if v not in ("bfloat16", "float32"):
                _fail(f"Error: '--dtype' got '{v}', expected bfloat16 or float32")
            g["dtype"] = v
            i += 2
        elif flag == "--std":
            g["std"] = _float_in(args, i, flag, 0.0, 10.0, "a number from 0 to 10")
            i += 2
        elif flag.startswith("-"):
            _fail(f"Error: unknown argument '{flag}'")
        elif g["config"] is None:
            g["config"] = flag
            i += 1
        elif g["out"] is None:
            g["out"] = flag
            i += 1
        else:
            _fail(f"Error: unexpected argument '{flag}'")
    if g["config"] is None or g["out"] is None:
        _fail("Error: 'hk random' needs a config.json (or a folder that holds one) and a folder to write")
    return g


def cmd_random(args) -> int:
    """Writes a model folder with seeded random weights of the architecture that a config.json names (no GPU)."""
    import os
    try:
        g = parse_random_args(args)
    except BadUsage as e:
        print(f"{e}\n{USAGE}", file=sys.stderr, end="")
        return 2
    import json
    import torch
    from .config import ConfigError, config_from_dict
    from .weights import write_random_model
    path = os.path.join(g["config"], "config.json") if os.path.isdir(g["config"]) else g["config"]
    try:
        with open(path, encoding="utf-8") as f:
            config = config_from_dict(json.load(f))
        if os.path.exists(os.path.join(g["out"], "model.safetensors")):
            print(f"Error: '{g['out']}' already holds a model.safetensors", file=sys.stderr)
            return 1
        write_random_model(g["out"], config, g["seed"], std=g["std"],
                           dtype=torch.float32 if g["dtype"] == "float32" else torch.bfloat16)
    except (ConfigError, FileNotFoundError, json.JSONDecodeError) as e:
        print(f"Error: {e}", file=sys.stderr)
        return 1
    print(f"wrote {g['out']} ({config.architecture}, seed {g['seed']}, {g['dtype']})", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(USAGE, end="")
        return 0 if argv else 2
    if argv[0] == "run":
        return cmd_run(argv[1:])
    if argv[0] == "random":
        return cmd_random(argv[1:])
    print(f"Error: unknown command '{argv[0]}' (this engine has 'run' and 'random')\n{USAGE}", file=sys.stderr, end="")
    return 2


if __name__ == "__main__":
    sys.exit(main())

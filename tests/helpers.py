"""Shared fixtures of the tests: the two tiny configurations, model folders with random
weights, a reader of safetensors that is independent of the engine's, and trace builders."""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

# Two tiny configurations that differ in every size and option.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=2,
    intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128,
    hidden_act="silu", attention_bias=False, initializer_range=0.02)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=96, num_hidden_layers=3,
    intermediate_size=320, num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=512,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256,
    hidden_act="silu", attention_bias=False, initializer_range=0.03)
# A third one for the windowed mixer and odd sizes: width and vocabulary that are no power of
# two nor a multiple of 16, five heads in one group, head size 48, a window on two of four layers.
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=72, num_hidden_layers=4,
    intermediate_size=200, num_attention_heads=5, num_key_value_heads=1, head_dim=48, vocab_size=333,
    rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=512,
    hidden_act="silu", attention_bias=False, initializer_range=0.05, partial_rotary_factor=0.5,
    use_sliding_window=True, sliding_window=20,
    layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"])

# Two more with the head sizes of real checkpoints (64 and 128), which take the TMA-fed decode attention and
# the widest flash tiles: D has 3 query heads per kv head and a window on its middle layer, E one kv head.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=136, num_hidden_layers=3,
    intermediate_size=264, num_attention_heads=6, num_key_value_heads=2, head_dim=64, vocab_size=777,
    rope_theta=250000.0, rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=1024,
    hidden_act="silu", attention_bias=False, initializer_range=0.04, use_sliding_window=True, sliding_window=70,
    layer_types=["full_attention", "sliding_attention", "full_attention"])
TINY_E = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=256, num_hidden_layers=2,
    intermediate_size=384, num_attention_heads=4, num_key_value_heads=1, head_dim=128, vocab_size=1000,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048,
    hidden_act="silu", attention_bias=False, initializer_range=0.03)

# F is built to miss every fast path: a width that is no multiple of 8 (the tensor-core products need that),
# plain multi-head attention (as many kv heads as heads) with the largest head size, an odd vocabulary.
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=100, num_hidden_layers=2,
    intermediate_size=148, num_attention_heads=3, num_key_value_heads=3, head_dim=256, vocab_size=1001,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=300,
    hidden_act="silu", attention_bias=False, initializer_range=0.02, partial_rotary_factor=0.25)

# G has a head size that is no multiple of 16 (the tensor-core attention refuses it; the generic kernels take it) and
# a rotary width of 24 of its 40.
TINY_G = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=88, num_hidden_layers=2,
    intermediate_size=136, num_attention_heads=4, num_key_value_heads=2, head_dim=40, vocab_size=401,
    rope_theta=20000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=256,
    hidden_act="silu", attention_bias=False, initializer_range=0.04, partial_rotary_factor=0.6)

TINY = {"G": (TINY_G, 9, 0.04, 0.1), "A": (TINY_A, 0, 0.02, 0.05), "B": (TINY_B, 1, 0.03, 0.1), "C": (TINY_C, 5, 0.05, 0.1),
        "D": (TINY_D, 6, 0.04, 0.1), "E": (TINY_E, 7, 0.03, 0.05), "F": (TINY_F, 8, 0.02, 0.05)}

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I32": np.int32, "I64": np.int64}


def read_safetensors(path: str) -> dict:
    """name -> float64/int numpy array; bfloat16 is widened exactly."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        base = 8 + hlen
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        if info["dtype"] == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=_ST_DTYPES[info["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(info["shape"])
    return out


def make_model_dir(tmpdir, which: str, dtype=torch.float32) -> str:
    """Writes tiny configuration `which` with its seed to a fresh folder; returns the path."""
    from hk_b200.config import config_from_dict
    from hk_b200.weights import write_random_model
    raw, seed, std, norm_std = TINY[which]
    d = os.path.join(str(tmpdir), f"tiny_{which}_{str(dtype).split('.')[-1]}")
    write_random_model(d, config_from_dict(raw), seed, std=std, norm_std=norm_std, dtype=dtype)
    return d


def load_plain(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


def prompts_for(which: str, rng: np.random.Generator, lengths):
    vocab = TINY[which][0]["vocab_size"]
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


# ---- traces: lists of steps {"entries": [(id, tokens, want)], "end": [ids]} -----------------


def trace_whole(seqs: dict):
    """Each request alone and whole, all places wanted."""
    steps = []
    for rid, ids in seqs.items():
        steps.append({"entries": [(rid, ids, list(range(len(ids))))], "end": [rid]})
    return steps


def trace_tail_decode(seqs: dict, tail: int = 32):
    """Most of each request in one step, then the last `tail` tokens one by one."""
    steps = []
    for rid, ids in seqs.items():
        head = max(1, len(ids) - tail)
        steps.append({"entries": [(rid, ids[:head], list(range(head)))], "end": []})
        for i in range(head, len(ids)):
            steps.append({"entries": [(rid, [ids[i]], [0])], "end": [rid] if i == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(seqs: dict, sizes=(13, 2, 7, 5, 31, 3, 2, 64, 1, 17)):
    """Portions of changing size, down to two tokens (and one)."""
    steps = []
    for rid, ids in seqs.items():
        pos, k = 0, 0
        while pos < len(ids):
            c = min(sizes[k % len(sizes)], len(ids) - pos)
            last = pos + c == len(ids)
            steps.append({"entries": [(rid, ids[pos:pos + c], list(range(c)))], "end": [rid] if last else []})
            pos += c
            k += 1
    return steps


def trace_mixed(seqs: dict, rng: np.random.Generator, max_live: int = 4, prefill_chunks=(13, 5, 2, 29, 8),
                decode_tail: int = 12):
    """Up to `max_live` live requests; portions of some beside single tokens of others.  A
    request is prefilled in portions until `decode_tail` tokens remain, which then come one by
    one, so decode rows and prompt portions share steps.  Requests wait until a slot is free, so
    with a small pool later requests get the pages earlier ones gave back."""
    waiting = list(seqs.items())
    live = {}   # rid -> [ids, pos]
    steps = []
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = [ids, 0]
        entries, end = [], []
        for rid in list(live):
            ids, pos = live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue    # this request sits the step out
            remain = len(ids) - pos
            if remain > decode_tail:
                c = min(prefill_chunks[k % len(prefill_chunks)], remain - decode_tail)
                k += 1
            else:
                c = 1
            entries.append((rid, ids[pos:pos + c], list(range(c))))
            live[rid][1] = pos + c
            if pos + c == len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def peak_tokens(steps, quantum: int = 64) -> int:
    """The most tokens live requests hold at any time, each request rounded up to `quantum`
    (requests ending after a step still hold their tokens during it)."""
    held, peak = {}, 0
    for st in steps:
        for rid, toks, _ in st["entries"]:
            held[rid] = held.get(rid, 0) + len(toks)
        peak = max(peak, sum(round_up(v, quantum) for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


def run_trace_on_engine(engine, steps):
    """Runs `steps` through an Engine; returns {(rid, position): logits row (numpy)}."""
    from hk_b200.engine import StepEntry
    got, pos = {}, {}
    for st in steps:
        entries = []
        for rid, toks, want in st["entries"]:
            if not engine.has_request(rid):
                engine.open_request(rid)
                pos[rid] = 0
            entries.append(StepEntry(rid, toks, want))
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.float().cpu().numpy()
            r = 0
            for rid, toks, want in st["entries"]:
                for w in want:
                    got[(rid, pos[rid] + w)] = arr[r]
                    r += 1
        for rid, toks, _ in st["entries"]:
            pos[rid] += len(toks)
        for rid in st["end"]:
            engine.close_request(rid)
            pos.pop(rid)
    return got


def trace_to_jsonl(steps) -> str:
    lines = []
    for i, st in enumerate(steps):
        lines.append(json.dumps({
            "step": i,
            "entries": [{"id": rid, "tokens": [int(t) for t in toks], "want": [int(w) for w in want]}
                        for rid, toks, want in st["entries"]],
            "end": list(st["end"])}))
    return "\n".join(lines) + "\n"

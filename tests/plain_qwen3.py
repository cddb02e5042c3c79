"""Plain, slow implementation of the Qwen3 dense decoder: the oracle of the test-suite.

It rests on the reference's formulas alone.  The reference's model code is Zig
(src/engine/*.zig) and no Zig toolchain exists where these tests run; its Python
package's pure-Python model is a LayerNorm/GELU toy (python/hk/modeling.py:298-350)
and not this architecture, so nothing of the reference can be executed to anchor
this file.  Every function below cites the lines it restates.

Rules of this file: whole sequences, no cache, no batching, one function for each
part, numpy only, and no import from the engine package.  Arithmetic is float64 by
default (`dtype=np.float64`), which makes it the common yardstick for the engine's
32-bit and bfloat16 paths; `dtype=np.float32` mimics the reference's own precision.
"""
from __future__ import annotations

import numpy as np


# --------------------------------------------------------------------------- parts


def embedding(table: np.ndarray, token_ids, dtype=np.float64) -> np.ndarray:
    """x[t, :] = E[token_t, :]  (src/engine/cpu_backend.zig:237-244)."""
    return table[np.asarray(token_ids, dtype=np.int64)].astype(dtype)


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """out = x / sqrt(mean(x^2) + eps) * w, mean over the last axis, eps inside the
    root, weight applied after normalising (src/engine/ops.zig:10-29)."""
    ss = np.mean(x * x, axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(ss + x.dtype.type(eps))
    return x * inv * weight.astype(x.dtype)


def head_norm(x: np.ndarray, weight: np.ndarray, head_dim: int, eps: float) -> np.ndarray:
    """Per-head RMS norm with one weight vector [head_dim] shared by every head
    (src/engine/ops.zig:32-38; order q then k, before RoPE: src/kernels_impl.zig:55-66)."""
    t, width = x.shape
    heads = width // head_dim
    return rms_norm(x.reshape(t, heads, head_dim), weight, eps).reshape(t, width)


def rope_inv_freq(theta: float, rotary_dim: int) -> np.ndarray:
    """inv_freq[i] = theta^(-2i/rotary_dim), derived in float64 and cast to float32
    (src/engine/ops.zig:96-144, kind `.none`)."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    return np.power(np.float64(theta), -(2.0 * i) / np.float64(rotary_dim)).astype(np.float32)


def rope_inv_freq_scaled(theta: float, rotary_dim: int, kind: str, factor: float = 1.0, orig_ctx: int = 0,
                         low_freq_factor: float = 1.0, high_freq_factor: float = 4.0, beta_fast: float = 32.0,
                         beta_slow: float = 1.0) -> np.ndarray:
    """Frequencies stretched for longer contexts (src/engine/ops.zig:96-144), every step in float64:
    linear: inv / factor; llama3: by wavelength against orig_ctx / high and orig_ctx / low with a blended
    band; yarn: a ramp between the dims that make beta_fast and beta_slow rotations in orig_ctx."""
    n = float(rotary_dim)
    out = np.zeros(rotary_dim // 2, dtype=np.float64)
    low = high = 0.0
    if kind == "yarn":
        corr = lambda rot: n * np.log(orig_ctx / (rot * 2.0 * np.pi)) / (2.0 * np.log(theta))
        low = max(0.0, np.floor(corr(beta_fast)))
        high = min(n - 1.0, np.ceil(corr(beta_slow)))
        if low == high:
            high += 0.001
    for i in range(rotary_dim // 2):
        inv = float(theta) ** (-(2.0 * i) / n)
        if kind == "none":
            v = inv
        elif kind == "linear":
            v = inv / factor
        elif kind == "llama3":
            wavelen = 2.0 * np.pi / inv
            if wavelen < orig_ctx / high_freq_factor:
                v = inv
            elif wavelen > orig_ctx / low_freq_factor:
                v = inv / factor
            else:
                smooth = (orig_ctx / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
                v = (1.0 - smooth) * inv / factor + smooth * inv
        elif kind == "yarn":
            ramp = min(1.0, max(0.0, (i - low) / (high - low)))
            v = (inv / factor) * ramp + inv * (1.0 - ramp)
        else:
            raise ValueError(kind)
        out[i] = v
    return out.astype(np.float32)


def rope_mscale(kind: str, factor: float = 1.0, attn_factor: float = 1.0) -> float:
    """Only yarn changes the magnitude: attn_factor * (0.1 ln(factor) + 1) (src/engine/ops.zig:146-151)."""
    return float(np.float32(attn_factor) * np.float32(1.0 + 0.1 * np.log(factor))) if kind == "yarn" else 1.0


def rope_rotate_adjacent(x: np.ndarray, head_dim: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """The `.norm` style: pairs (2i, 2i + 1) over the first 2*len(cos) dims of every head
    (src/engine/ops.zig:166-172)."""
    t, width = x.shape
    heads = width // head_dim
    half = cos.shape[1]
    xr = x.reshape(t, heads, head_dim).copy()
    a = xr[:, :, 0:2 * half:2].copy()
    b = xr[:, :, 1:2 * half:2].copy()
    c = cos[:, None, :].astype(x.dtype)
    s = sin[:, None, :].astype(x.dtype)
    xr[:, :, 0:2 * half:2] = a * c - b * s
    xr[:, :, 1:2 * half:2] = a * s + b * c
    return xr.reshape(t, width)


def rope_angles(positions, inv_freq: np.ndarray):
    """a = f32(pos) * inv_freq[i] in float32; cos and sin of that float32 angle
    (src/engine/ops.zig:154-161; mscale is 1 without YaRN, ops.zig:146-151)."""
    p = np.asarray(positions, dtype=np.float32)[:, None]
    a = (p * inv_freq[None, :]).astype(np.float32)
    a64 = a.astype(np.float64)
    return np.cos(a64), np.sin(a64)


def rope_rotate_half(x: np.ndarray, head_dim: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half ("neox") pairing over the first 2*len(cos) dims of every head:
    x'[i] = x[i] c - x[i+half] s ; x'[i+half] = x[i] s + x[i+half] c
    (src/engine/ops.zig:176-181; HF imports are always neox: src/convert/hf.zig:312)."""
    t, width = x.shape
    heads = width // head_dim
    half = cos.shape[1]
    xr = x.reshape(t, heads, head_dim).copy()
    a = xr[:, :, :half].copy()
    b = xr[:, :, half:2 * half].copy()
    c = cos[:, None, :].astype(x.dtype)
    s = sin[:, None, :].astype(x.dtype)
    xr[:, :, :half] = a * c - b * s
    xr[:, :, half:2 * half] = a * s + b * c
    return xr.reshape(t, width)


def causal_gqa_attention(q, k, v, n_heads, n_kv_heads, head_dim, window=None, kv_round=None):
    """Causal grouped-query attention over a whole sequence.

    scale = 1/sqrt(head_dim) applied to q first (src/engine/attention.zig:90,
    src/engine/attention_kernel.zig:109); q head h reads kv head h // (H/G)
    (attention.zig:56, src/cuda_device.zig:1510); the token at position p sees
    j in [0, p] (attention_kernel.zig:112,214-220); softmax in the working precision
    (attention_kernel.zig:223-249); out = sum_j p_j v_j / sum_j p_j (:149-156,252-279).

    `window` (not a reference feature: the reference refuses sliding windows,
    src/engine/config.zig:271-279) limits j to (p - window, p]; it serves the tests of
    the general attention part.  `kv_round` optionally rounds k and v the way a cache
    of reduced precision stores them (the reference stores float16: src/engine/kv.zig:125-134).
    """
    t = q.shape[0]
    group = n_heads // n_kv_heads
    if kv_round is not None:
        k = kv_round(k)
        v = kv_round(v)
    qh = q.reshape(t, n_heads, head_dim) * q.dtype.type(1.0 / np.sqrt(np.float64(head_dim)))
    kh = k.reshape(t, n_kv_heads, head_dim)
    vh = v.reshape(t, n_kv_heads, head_dim)
    out = np.zeros((t, n_heads, head_dim), dtype=q.dtype)
    pos = np.arange(t)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > pos[:, None] - window
    for h in range(n_heads):
        g = h // group
        s = qh[:, h, :] @ kh[:, g, :].T
        s = np.where(visible, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        p = np.exp(s - m)
        out[:, h, :] = (p @ vh[:, g, :]) / p.sum(axis=-1, keepdims=True)
    return out.reshape(t, n_heads * head_dim)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = x W^T with W stored [out, in] (src/engine/matmul.zig:5,23; no bias for
    qwen3: src/engine/config.zig:313)."""
    return x @ w.astype(x.dtype).T


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """h = g / (1 + exp(-g)) * u  (src/engine/ops.zig:65-80)."""
    return gate / (1.0 + np.exp(-gate)) * up


# --------------------------------------------------------------------------- model


def _cfg(cfg: dict, key: str, default=None):
    v = cfg.get(key, default)
    return default if v is None else v


def forward(cfg: dict, weights: dict, token_ids, dtype=np.float64, kv_round=None,
            act_round=None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence starting at position 0.

    `cfg` holds config.json's keys; `weights` maps Hugging Face tensor names to numpy
    arrays.  Layer order follows src/engine/cpu_backend.zig:258-325; the head follows
    :329-357 and the tied-output rule src/engine/weights.zig:124-129.
    `act_round`, when given, rounds the input of every matrix product (how a
    reduced-precision engine feeds its tensor cores); the residual stays unrounded.
    """
    d = cfg["hidden_size"]
    n_heads = cfg["num_attention_heads"]
    n_kv = _cfg(cfg, "num_key_value_heads", n_heads)            # src/convert/hf.zig:272
    hd = _cfg(cfg, "head_dim", d // n_heads)                    # src/convert/hf.zig:273
    eps = float(_cfg(cfg, "rms_norm_eps", 1e-6))                # src/convert/hf.zig:293
    theta = float(_cfg(cfg, "rope_theta", 10000.0))             # src/convert/hf.zig:294
    rot = int(hd * float(_cfg(cfg, "partial_rotary_factor", 1.0)))   # src/convert/hf.zig:299-300
    n_layers = cfg["num_hidden_layers"]
    windows = layer_windows(cfg)
    rnd = act_round if act_round is not None else (lambda a: a)

    t = len(token_ids)
    x = embedding(weights["model.embed_tokens.weight"], token_ids, dtype)
    cos, sin = rope_angles(np.arange(t), rope_inv_freq(theta, rot))
    for li in range(n_layers):
        p = f"model.layers.{li}."
        xb = rnd(rms_norm(x, weights[p + "input_layernorm.weight"], eps))
        q = linear(xb, weights[p + "self_attn.q_proj.weight"])
        k = linear(xb, weights[p + "self_attn.k_proj.weight"])
        v = linear(xb, weights[p + "self_attn.v_proj.weight"])
        q = head_norm(q, weights[p + "self_attn.q_norm.weight"], hd, eps)
        k = head_norm(k, weights[p + "self_attn.k_norm.weight"], hd, eps)
        q = rnd(rope_rotate_half(q, hd, cos, sin))
        k = rope_rotate_half(k, hd, cos, sin)
        att = causal_gqa_attention(q, k, v, n_heads, n_kv, hd, window=windows[li], kv_round=kv_round)
        x = x + linear(rnd(att), weights[p + "self_attn.o_proj.weight"])
        xb = rnd(rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps))
        h = swiglu(linear(xb, weights[p + "mlp.gate_proj.weight"]),
                   linear(xb, weights[p + "mlp.up_proj.weight"]))
        x = x + linear(rnd(h), weights[p + "mlp.down_proj.weight"])
    xb = rnd(rms_norm(x, weights["model.norm.weight"], eps))
    head = weights.get("lm_head.weight")
    if head is None:
        if not _cfg(cfg, "tie_word_embeddings", False):
            raise KeyError("lm_head.weight is absent and tie_word_embeddings is false")
        head = weights["model.embed_tokens.weight"]
    return linear(xb, head)


def layer_windows(cfg: dict):
    """Per-layer window (None = all keys).  The reference itself has no windowed
    Qwen3 (src/convert/hf.zig:256-262 refuses it); the engine accepts config.json's
    `layer_types` / `use_sliding_window` keys, so the oracle mirrors that reading."""
    n = cfg["num_hidden_layers"]
    w = cfg.get("sliding_window")
    if not cfg.get("use_sliding_window", False) or not w:
        return [None] * n
    types = cfg.get("layer_types")
    if types is None:
        mwl = cfg.get("max_window_layers", n)
        types = ["sliding_attention" if i >= mwl else "full_attention" for i in range(n)]
    return [int(w) if ty == "sliding_attention" else None for ty in types]


# --------------------------------------------------------------------------- sampling


def greedy(logits: np.ndarray) -> int:
    """First maximum wins (src/sampler.zig:128-135)."""
    return int(np.argmax(logits))


def candidate_distribution(logits: np.ndarray, temperature: float, top_k: int, top_p: float,
                           min_p: float = 0.0, max_candidates: int = 4096):
    """The reference's chain (src/sampler.zig:137-204): top-k (0 = capped at 4096)
    sorted by logit desc and id asc, probabilities at temperature 1 for top-p (keep
    through the first that reaches p) and min-p, then temperature on the survivors.
    Returns (ids, probabilities) of the survivors, normalised."""
    logits = np.asarray(logits, dtype=np.float64)
    ids = np.arange(len(logits))
    finite = np.isfinite(logits)
    ids, vals = ids[finite], logits[finite]
    order = np.lexsort((ids, -vals))
    k = min(top_k if top_k > 0 else max_candidates, max_candidates, len(order))
    order = order[:k]
    ids, vals = ids[order], vals[order]
    p = np.exp(vals - vals[0])
    p /= p.sum()
    keep = len(ids)
    if 0 < top_p < 1:
        cum = np.cumsum(p)
        hit = np.nonzero(cum >= top_p)[0]
        if len(hit):
            keep = int(hit[0]) + 1
    if min_p > 0:
        floor = p[0] * min_p
        i = 0
        while i < keep and p[i] >= floor:
            i += 1
        keep = max(1, i)
    w = np.exp((vals[:keep] - vals[0]) / temperature)
    return ids[:keep], w / w.sum()

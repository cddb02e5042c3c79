"""Python face of the CUDA kernels: argument checks, kernel choice, launch on torch's
current stream.

Every function takes torch CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes) and raises `KernelError` with a clear message when a kernel refuses a
shape; nothing falls back to the CPU or to a library.  Kernel choice (tensor-core GEMM or
generic GEMM, flash or generic attention) is by shape alone, never by batch content, and
can be pinned with `force()` by tests.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_ERR_UNSUPPORTED = 100001


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, not {t.dim()}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """How many kernel launches this module has issued so far (for benchmarks' bookkeeping)."""
    return _launches


def count_launches(n: int) -> None:
    """Adds kernel launches made outside this module's wrappers (a replayed CUDA graph's nodes)."""
    global _launches
    _launches += n


def _check(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code == _ERR_UNSUPPORTED:
        raise KernelError(f"{what}: the kernel refuses these sizes or types")
    raise KernelError(f"{what}: CUDA error {code}")


# ---- kernel choice --------------------------------------------------------------------

_forced = {"gemm": None, "attention": None}


def forced(kind: str) -> Optional[str]:
    """The kernel family pinned for `kind` ('gemm' or 'attention'), or None."""
    return _forced[kind]


@contextlib.contextmanager
def force(gemm: Optional[str] = None, attention: Optional[str] = None):
    """Pins the kernel family inside the block: gemm in {'generic','tc','smallm','stream'},
    attention in {'generic','flash','flash_cp'} ('flash_cp': the flash kernels without the TMA-fed decode
    variant).  A pinned kernel that refuses the shape raises."""
    old = dict(_forced)
    if gemm is not None:
        _forced["gemm"] = gemm
    if attention is not None:
        _forced["attention"] = attention
    try:
        yield
    finally:
        _forced.update(old)


# ---- embedding ------------------------------------------------------------------------


def embedding(table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = table[token_ids[t], :] widened to float32."""
    _need(table, "table", dims=2)
    _need(token_ids, "token_ids", torch.int32, 1)
    _need(out, "out", torch.float32, 2)
    n, d = out.shape
    if token_ids.shape[0] != n or table.shape[1] != d:
        raise KernelError(f"embedding: out {tuple(out.shape)} does not fit ids {tuple(token_ids.shape)} and table {tuple(table.shape)}")
    lib = build.load("elementwise")
    _check(lib.hk_embedding(_ptr(table), _dt(table), _ptr(token_ids), _ptr(out), n, d, table.shape[0], _stream()),
           "embedding")


# ---- rms norm -------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = x[rows[r] or r, :] * rsqrt(mean(x^2) + eps) * weight  (x, weight float32)."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dims=2)
    d = x.shape[1]
    n_out = out.shape[0]
    if weight.shape[0] != d or out.shape[1] != d:
        raise KernelError("rms_norm: widths of x, weight and out differ")
    if rows is None:
        if n_out != x.shape[0]:
            raise KernelError("rms_norm: out has other rows than x")
    else:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] < n_out:
            raise KernelError("rms_norm: fewer row indices than output rows")
    lib = build.load("elementwise")
    _check(lib.hk_rms_norm(_ptr(x), _ptr(weight), _ptr(rows), _ptr(out), _dt(out), n_out, d,
                           ctypes.c_float(eps), _stream()), "rms_norm")


# ---- swiglu ---------------------------------------------------------------------------


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[t, j] = silu(gate) * up for gate_up float32 [n, 2F].  With block = 0 the row is laid out
    [F gates | F ups]; with block = b (dividing F) it is [b gates | b ups | b gates | ...]."""
    _need(gate_up, "gate_up", torch.float32, 2)
    _need(out, "out", dims=2)
    n, f = out.shape
    block = block or f
    if gate_up.shape[0] != n or gate_up.shape[1] != 2 * f or f % block:
        raise KernelError("swiglu: gate_up must be [n, 2F] for out [n, F], and the block must divide F")
    lib = build.load("elementwise")
    _check(lib.hk_swiglu(_ptr(gate_up), _ptr(out), _dt(out), n, f, int(block), _stream()), "swiglu")


def _as_weights(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """A product runs in its weights' type: where a matrix is kept in 32-bit although the engine computes in
    bfloat16 (its file stored it so), the activations are widened for that product (and narrowed for the next)."""
    if a.dtype == w.dtype:
        return a
    if w.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"weights must be float32 or bfloat16, not {w.dtype}")
    return a.to(w.dtype)


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, F] = silu(gate) * up of a @ w_gate_up^T, w_gate_up [2F, K] = [F gate rows | F up rows].  Fused into
    the tensor-core product's epilogue when that takes the shape (a tile of the product then holds gate rows and
    the up rows that match them), else a product to float32 followed by the swiglu kernel."""
    _need(a, "a", dims=2)
    _need(w_gate_up, "w", dims=2)
    _need(out, "out", a.dtype, 2)
    if w_gate_up.dtype != a.dtype:              # weights kept in 32-bit on the bfloat16 path: this product runs in 32-bit
        wide = torch.empty(out.shape, dtype=w_gate_up.dtype, device=out.device)
        gemm_swiglu(_as_weights(a, w_gate_up), w_gate_up, wide)
        out.copy_(wide)
        return
    M, F = out.shape
    if a.shape[0] != M or w_gate_up.shape != (2 * F, a.shape[1]):
        raise KernelError("gemm_swiglu: shapes do not fit")
    if a.dtype == torch.bfloat16 and _forced["gemm"] in (None, "tc", "stream"):
        from . import gemm_fast
        if gemm_fast.run_swiglu(a, w_gate_up, out, _forced["gemm"]):
            return
    gu = torch.empty((M, 2 * F), dtype=torch.float32, device=a.device)
    gemm(a, w_gate_up, gu)
    swiglu(gu, out, 0)


# ---- per-head norm + rotation + cache write ---------------------------------------------


PAIRINGS = {"half": 0, "adjacent": 1}


def qk_norm_rope_kv_write(qkv, q_out, q_weight, k_weight, eps, cos, sin, rotary_dim, positions,
                          slot_of_token, block_table, k_pages, v_pages, n_heads, n_kv_heads, head_dim,
                          page_tokens, write_kv=True, bias=None, pairing="half") -> None:
    """Splits the fused projection qkv[n, (H+2G)*hd] (float32): q heads are normalised (if
    q_weight), rotated (if rotary_dim > 0) and stored to q_out[n, H*hd]; k heads likewise and
    stored, with the v heads, into the token's cache page [page, G, page_tokens, hd].
    `bias` (float32 [(H+2G)*hd]) is added to the projection first.  `pairing`: "half" rotates dims
    (i, i + rotary_dim/2), "adjacent" dims (2i, 2i+1)."""
    if pairing not in PAIRINGS:
        raise KernelError(f"qk_norm_rope_kv_write: pairing {pairing!r} is neither 'half' nor 'adjacent'")
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != (n_heads + 2 * n_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_kv_write: bias must have (H + 2G) * head_dim entries")
    _need(qkv, "qkv", torch.float32, 2)
    _need(q_out, "q_out", dims=2)
    n = qkv.shape[0]
    H, G, hd = n_heads, n_kv_heads, head_dim
    if qkv.shape[1] != (H + 2 * G) * hd or tuple(q_out.shape) != (n, H * hd):
        raise KernelError("qk_norm_rope_kv_write: qkv or q_out has the wrong shape")
    if head_dim > 256:
        raise KernelError(f"qk_norm_rope_kv_write: head_dim {head_dim} is above 256")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _need(w, name, torch.float32, 1)
            if w.shape[0] != hd:
                raise KernelError(f"{name} must have head_dim entries")
    if rotary_dim > 0:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape or rotary_dim % 2 or rotary_dim > hd:
            raise KernelError("rotation tables must be [positions, rotary_dim/2]")
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    if write_kv:
        _need(block_table, "block_table", torch.int32, 2)
        _need(k_pages, "k_pages", q_out.dtype, 4)
        _need(v_pages, "v_pages", q_out.dtype, 4)
        if tuple(k_pages.shape[1:]) != (G, page_tokens, hd) or k_pages.shape != v_pages.shape:
            raise KernelError("cache pages must be [pages, G, page_tokens, head_dim]")
    lib = build.load("elementwise")
    _check(lib.hk_qk_norm_rope_kv_write(
        _ptr(qkv), _ptr(q_out), _dt(q_out), _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps),
        _ptr(cos if rotary_dim > 0 else None), _ptr(sin if rotary_dim > 0 else None), int(rotary_dim),
        _ptr(positions), _ptr(slot_of_token), _ptr(block_table if write_kv else None),
        int(block_table.shape[1]) if write_kv else 0, _ptr(k_pages if write_kv else None),
        _ptr(v_pages if write_kv else None), n, H, G, hd, int(page_tokens), 1 if write_kv else 0, _ptr(bias),
        PAIRINGS[pairing], _stream()),
        "qk_norm_rope_kv_write")


# ---- matrix product -------------------------------------------------------------------


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[t, :] += bias (both float32)."""
    _need(out, "out", torch.float32, 2)
    _need(bias, "bias", torch.float32, 1)
    if bias.shape[0] != out.shape[1]:
        raise KernelError("add_bias: one bias entry per output column")
    lib = build.load("elementwise")
    _check(lib.hk_add_bias(_ptr(out), _ptr(bias), out.shape[0], out.shape[1], _stream()), "add_bias")


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
         bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] (float32) = a[M, K] @ w[N, K]^T (+ out when `accumulate`) (+ bias[N], float32).
    a and w share a type: float32 (plain FMA) or bfloat16 (fp32 accumulation)."""
    if bias is not None:
        gemm(a, w, out, accumulate)
        add_bias(out, bias)
        return
    _need(a, "a", dims=2)
    _need(w, "w", dims=2)
    _need(out, "out", torch.float32, 2)
    a = _as_weights(a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    choice = _forced["gemm"]
    if a.dtype == torch.bfloat16 and choice != "generic":
        from . import gemm_fast
        if gemm_fast.run(a, w, out, accumulate, choice):
            return
        if choice is not None:
            raise KernelError(f"gemm: the '{choice}' kernel refuses M={M} N={N} K={K}")
    lib = build.load("gemm_generic")
    _check(lib.hk_gemm_generic(_ptr(a), _ptr(w), _dt(a), _ptr(out), M, N, K, ctypes.c_longlong(K),
                               ctypes.c_longlong(K), ctypes.c_longlong(N), 1 if accumulate else 0, _stream()),
           "gemm")


# ---- attention ------------------------------------------------------------------------


def paged_attention(q, k_pages, v_pages, block_table, positions, slot_of_token, out, n_heads, n_kv_heads,
                    head_dim, page_tokens, window: int, scale: float, plan=None) -> None:
    """out[t, h, :] = softmax_j(scale * q[t, h] . k[j]) v[j] over the keys j in
    [max(0, p - window + 1), p] (all of [0, p] when window <= 0) of the token's request, read
    through its block-table row; p = positions[t].  `plan` carries the per-request tiling the
    flash kernel wants; without it (or for sizes it refuses) the generic kernel runs."""
    _need(q, "q", dims=2)
    _need(out, "out", q.dtype, 2)
    _need(k_pages, "k_pages", q.dtype, 4)
    _need(v_pages, "v_pages", q.dtype, 4)
    _need(block_table, "block_table", torch.int32, 2)
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    n = q.shape[0]
    H, G, hd = n_heads, n_kv_heads, head_dim
    if tuple(q.shape) != (n, H * hd) or out.shape != q.shape:
        raise KernelError("paged_attention: q and out must be [n, H*head_dim]")
    if tuple(k_pages.shape[1:]) != (G, page_tokens, hd) or k_pages.shape != v_pages.shape:
        raise KernelError("paged_attention: cache pages must be [pages, G, page_tokens, head_dim]")
    if H % G != 0:
        raise KernelError(f"paged_attention: {H} heads are not a multiple of {G} groups")
    if hd > 256:
        raise KernelError(f"paged_attention: head_dim {hd} is above 256")
    choice = _forced["attention"]
    if q.dtype == torch.bfloat16 and choice != "generic" and plan is not None:
        from . import attention_fast
        if attention_fast.run(q, k_pages, v_pages, block_table, out, H, G, hd, page_tokens, window, scale, plan,
                              allow_tma=choice != "flash_cp"):
            return
        if choice is not None:
            raise KernelError(f"paged_attention: the '{choice}' kernel refuses head_dim={hd} page_tokens={page_tokens}")
    lib = build.load("attention_generic")
    _check(lib.hk_attention_generic(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _dt(q), _ptr(block_table), int(block_table.shape[1]),
        _ptr(positions), _ptr(slot_of_token), _ptr(out), n, H, G, hd, int(page_tokens), int(window),
        ctypes.c_float(scale), _stream()), "paged_attention")


# ---- sampling -------------------------------------------------------------------------


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r, :] (float32)."""
    _need(logits, "logits", torch.float32, 2)
    _need(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax: one output per row")
    lib = build.load("sampling")
    _check(lib.hk_argmax(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _stream()), "argmax")


def adjust_logits(logits, offsets, ids, counts, bias, repeat_penalty, freq_penalty, presence_penalty) -> None:
    """Applies repetition, frequency and presence penalties and logit biases in place: entries
    offsets[r]..offsets[r+1] of (ids, counts, bias) belong to row r."""
    _need(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt, n in (("offsets", offsets, torch.int32, rows + 1), ("ids", ids, torch.int32, None),
                           ("counts", counts, torch.int32, ids.shape[0]), ("bias", bias, torch.float32, ids.shape[0]),
                           ("repeat_penalty", repeat_penalty, torch.float32, rows),
                           ("freq_penalty", freq_penalty, torch.float32, rows),
                           ("presence_penalty", presence_penalty, torch.float32, rows)):
        _need(t, name, dt, 1)
        if n is not None and t.shape[0] != n:
            raise KernelError(f"adjust_logits: {name} has {t.shape[0]} entries, expected {n}")
    lib = build.load("sampling")
    _check(lib.hk_adjust_logits(_ptr(logits), rows, logits.shape[1], _ptr(offsets), _ptr(ids), _ptr(counts), _ptr(bias),
                                _ptr(repeat_penalty), _ptr(freq_penalty), _ptr(presence_penalty), _stream()),
           "adjust_logits")


def sample(logits, temperature, top_k, top_p, min_p, seeds, counters, out) -> None:
    """One token per row by the chain top-k -> top-p -> min-p -> temperature -> draw; rows with
    temperature <= 0 take the first maximum.  seeds and counters are int64 per row."""
    _need(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int64), ("out", out, torch.int32)):
        _need(t, name, dt, 1)
        if t.shape[0] != rows:
            raise KernelError(f"sample: {name} must have one entry per row")
    lib = build.load("sampling")
    _check(lib.hk_sample(_ptr(logits), rows, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
                         _ptr(seeds), _ptr(counters), _ptr(out), _stream()), "sample")

"""Plain PyTorch float32/float64 references of the single kernels, for the kernel tests.

Each function restates one kernel's contract on CPU tensors, with the cache in the same
paged layout the kernel reads ([page, kv_head, page_tokens, head_dim] and a block table),
and shares no code with the engine package.  Formula sources are cited per function.
"""
from __future__ import annotations

import math

import torch


def embedding(table, token_ids):
    """x[t] = E[id_t] as float32 (src/engine/cpu_backend.zig:237-244)."""
    return table.float()[token_ids.long()]


def rms_norm(x, weight, eps, rows=None):
    """src/engine/ops.zig:10-29."""
    x = x.double()
    if rows is not None:
        x = x[rows.long()]
    inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    return x * inv * weight.double()


def swiglu(gate_up):
    """src/engine/ops.zig:65-80 on the fused [n, 2F] layout (gate | up)."""
    f = gate_up.shape[1] // 2
    g, u = gate_up[:, :f].double(), gate_up[:, f:].double()
    return g / (1.0 + torch.exp(-g)) * u


def gemm(a, w, out0=None):
    """y = a W^T (src/engine/matmul.zig:5,23), plus what the output held when accumulating."""
    y = a.double() @ w.double().T
    return y if out0 is None else y + out0.double()


def qk_norm_rope(qkv, q_weight, k_weight, eps, cos, sin, rotary_dim, positions, H, G, hd, bias=None, pairing="half"):
    """Per-head norm then rotation of the q and k heads of qkv[n, (H+2G)*hd]
    (src/engine/ops.zig:32-38; order: src/kernels_impl.zig:55-66); the rotation pairs dims
    (i, i + half) ("half", the reference's .neox) or (2i, 2i + 1) ("adjacent", its .norm):
    src/engine/ops.zig:164-181.  A bias is added to the projection first (cf. qkv_bias,
    src/engine/config.zig:313).  Returns q[n, H, hd], k[n, G, hd], v[n, G, hd] in float64."""
    n = qkv.shape[0]
    x = qkv.double()
    if bias is not None:
        x = x + bias.double()[None, :]
    x = x.reshape(n, H + 2 * G, hd)
    q, k, v = x[:, :H].clone(), x[:, H:H + G].clone(), x[:, H + G:].clone()

    def norm(t, w):
        if w is None:
            return t
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.double()

    def rope(t):
        if rotary_dim == 0:
            return t
        half = rotary_dim // 2
        c = cos.double()[positions.long()][:, None, :]
        s = sin.double()[positions.long()][:, None, :]
        t = t.clone()
        if pairing == "adjacent":
            a, b = t[..., 0:2 * half:2].clone(), t[..., 1:2 * half:2].clone()
            t[..., 0:2 * half:2] = a * c - b * s
            t[..., 1:2 * half:2] = a * s + b * c
            return t
        a, b = t[..., :half].clone(), t[..., half:2 * half].clone()
        t[..., :half] = a * c - b * s
        t[..., half:2 * half] = a * s + b * c
        return t

    return rope(norm(q, q_weight)), rope(norm(k, k_weight)), v


def write_pages(k, v, k_pages, v_pages, block_table, slot_of_token, positions, page_tokens):
    """Stores k, v [n, G, hd] at each token's (page, offset) (cf. kv_write, src/cuda_device.zig:1453-1477)."""
    for t in range(k.shape[0]):
        pos = int(positions[t])
        page = int(block_table[int(slot_of_token[t]), pos // page_tokens])
        k_pages[page, :, pos % page_tokens, :] = k[t].to(k_pages.dtype)
        v_pages[page, :, pos % page_tokens, :] = v[t].to(v_pages.dtype)


def paged_attention(q, k_pages, v_pages, block_table, positions, slot_of_token, H, G, hd, page_tokens,
                    window, scale):
    """Token at position p reads keys max(0, p-window+1)..p (window <= 0: 0..p) of its slot
    (src/engine/attention.zig:45-103; mask src/engine/attention_kernel.zig:112,214-220)."""
    n = q.shape[0]
    out = torch.zeros(n, H, hd, dtype=torch.float64)
    qh = q.double().reshape(n, H, hd) * scale
    group = H // G
    for t in range(n):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window > 0 else 0
        js = torch.arange(lo, p + 1)
        pages = block_table[int(slot_of_token[t])].long()[js // page_tokens]
        keys = k_pages[pages, :, js % page_tokens, :].double()      # [j, G, hd]
        vals = v_pages[pages, :, js % page_tokens, :].double()
        for h in range(H):
            s = keys[:, h // group, :] @ qh[t, h]
            w = torch.softmax(s, dim=0)
            out[t, h] = w @ vals[:, h // group, :]
    return out.reshape(n, H * hd)

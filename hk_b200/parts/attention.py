"""Grouped-query attention over a paged cache, as a mixer part.

Steps, in the reference's order (src/engine/cpu_backend.zig:266-304):
  q, k, v = xb Wq^T, xb Wk^T, xb Wv^T   (one fused product; no bias: src/engine/config.zig:313)
  per-head RMS norm of q and of k with a weight [head_dim] shared by the heads, before the
  rotation (src/engine/ops.zig:32-38, src/kernels_impl.zig:55-66) - optional here
  rotate-half rotation of q and k by position (src/engine/ops.zig:176-181) - optional here
  the step's k and v go to the cache before any score is taken (cpu_backend.zig:290-295)
  scores scale * q . k_j over the visible keys, softmax in float32, weighted values
  (src/engine/attention.zig:45-103), q head h reading kv head h // (H/G) (attention.zig:56)
  residual += att Wo^T (cpu_backend.zig:303-304)

Sizes, the norm's eps, the position encoding (with its pairing of dims), the window, the scale and
biases on the projections are parameters.  The
reference's attention has no window (src/engine/config.zig:271-279 refuses one); `window=w`
limits the keys of position p to (p - w, p] and lets the cache give pages back.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KVCacheSpec, MATRIX, VECTOR, ParamSpec, Part, Precision, StepTables, register_part
from .position import RotaryEmbedding


class GQAAttention(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, prefix: str,
                 qk_norm_eps: Optional[float] = None, position: Optional[RotaryEmbedding] = None,
                 window: Optional[int] = None, scale: Optional[float] = None, qkv_bias: bool = False,
                 o_bias: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim > 256 or head_dim < 2:
            raise ValueError(f"head_dim {head_dim} is outside 2..256")
        if position is not None and position.rotary_dim > head_dim:
            raise ValueError("the rotary width exceeds head_dim")
        self.hidden, self.H, self.G, self.hd = hidden, n_heads, n_kv_heads, head_dim
        self.prefix = prefix
        self.qk_norm_eps = qk_norm_eps
        self.position = position
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # biases on the projections: the reference turns `qkv_bias` on by architecture (src/engine/config.zig:313)
        self.qkv_bias, self.o_bias = bool(qkv_bias), bool(o_bias)
        self.b_qkv = self.b_o = None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self._tables_key = None        # set at bind: the flash kernels' work items, when they take these sizes
        self._sm_count = 0

    # -- declaration ---------------------------------------------------------------------
    def children(self):
        return (self.position,) if self.position is not None else ()

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, H, G, hd, d = self.prefix, self.H, self.G, self.hd, self.hidden
        specs = {
            p + "q_proj.weight": ParamSpec((H * hd, d), MATRIX),
            p + "k_proj.weight": ParamSpec((G * hd, d), MATRIX),
            p + "v_proj.weight": ParamSpec((G * hd, d), MATRIX),
            p + "o_proj.weight": ParamSpec((d, H * hd), MATRIX),
        }
        if self.qk_norm_eps is not None:
            specs[p + "q_norm.weight"] = ParamSpec((hd,), VECTOR, "one_plus_normal")
            specs[p + "k_norm.weight"] = ParamSpec((hd,), VECTOR, "one_plus_normal")
        if self.qkv_bias:
            specs[p + "q_proj.bias"] = ParamSpec((H * hd,), VECTOR)
            specs[p + "k_proj.bias"] = ParamSpec((G * hd,), VECTOR)
            specs[p + "v_proj.bias"] = ParamSpec((G * hd,), VECTOR)
        if self.o_bias:
            specs[p + "o_proj.bias"] = ParamSpec((d,), VECTOR)
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.G, self.hd, self.window)

    def own_bind(self, tensors, precision: Precision) -> None:
        p = self.prefix
        qkv = [tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"], tensors[p + "v_proj.weight"]]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in qkv) else qkv[0].dtype    # one kept in 32-bit: all are
        self.w_qkv = torch.cat([t.to(wide) for t in qkv], dim=0).contiguous()
        self.w_o = tensors[p + "o_proj.weight"]
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[p + f"{n}_proj.bias"] for n in "qkv"]).contiguous()
        if self.o_bias:
            self.b_o = tensors[p + "o_proj.bias"]
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[p + "q_norm.weight"]
            self.k_norm = tensors[p + "k_norm.weight"]
        from ..csrc import attention_fast
        if precision.compute == torch.bfloat16 and attention_fast.supported(self.hd, self.H // self.G):
            self._tables_key = ("paged_attention_items", self.window or 0, self.H, self.G, self.hd)
            self._sm_count = torch.cuda.get_device_properties(precision.device).multi_processor_count

    # -- the step's work items (host-built; see parts.base) --------------------------------
    def step_tables_key(self):
        return self._tables_key

    def step_tables(self, ctx):
        """Cuts the batch into the flash kernels' work items (csrc/attention_fast.py).  In a step whose shape must
        not change (a captured decode graph) every request's keys go to the same number of splits."""
        from ..csrc import attention_fast
        H, G, hd = self.H, self.G, self.hd
        tc = attention_fast.tc_prefill_supported(hd, H // G) and ops.forced("attention") != "flash_cp"
        rows = 128 if tc else 64
        # the kernel with two query tiles per CTA is the faster one per row, but halves the number of work items: it
        # is taken when its items still fill the SMs (measured on the 8B layer: equal at 1,024 prompt tokens = 128
        # items, 1.6 times faster at 2,048, 1.3 times slower at 512), where the pages allow it
        if tc and attention_fast.tc2_prefill_supported(hd, H // G, ctx.page_tokens):
            group = H // G
            items = G * sum(-(-(int(q) * group) // 256) for q in ctx.q_lens if int(q) * group > 128)
            if items * 20 >= self._sm_count * 17:
                rows = 256
        fixed = attention_fast.decode_splits(ctx.n_tokens, G, self._sm_count) if ctx.fixed_shape else 0
        got = attention_fast.plan_arrays(ctx.slots, ctx.q_starts, ctx.q_lens, ctx.start_positions, ctx.n_tokens,
                                         self.window or 0, H, G, self._sm_count, fixed_splits=fixed,
                                         max_context=ctx.max_context if ctx.fixed_shape else 0,
                                         prefill_rows=rows)
        if got is None:
            return None
        items, merge, info = got
        arrays = {"items": items}
        if merge is not None:
            arrays["merge"] = merge
        return StepTables(arrays, info)

    def _plan(self, ctx):
        got = ctx.tables.get(self._tables_key) if self._tables_key is not None else None
        if got is None or got[1] is None:
            return None                    # no work items: the generic kernel takes the step
        from ..csrc import attention_fast
        arrays, info = got
        return attention_fast.plan_on_device(info, arrays["items"], arrays.get("merge"))

    # -- one step ------------------------------------------------------------------------
    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True) -> None:
        n = xb.shape[0]
        H, G, hd = self.H, self.G, self.hd
        plan = self._plan(ctx) if xb.dtype == torch.bfloat16 else None
        qkv = torch.empty((n, (H + 2 * G) * hd), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_qkv, qkv)
        q = torch.empty((n, H * hd), dtype=xb.dtype, device=xb.device)
        cos = sin = None
        rot = 0
        pairing = "half"
        if self.position is not None:
            cos, sin, rot = self.position.tables()
            pairing = getattr(self.position, "pairing", "half")
        # the projections' bias rides on the fused kernel's load
        ops.qk_norm_rope_kv_write(
            qkv, q, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, cos, sin, rot, ctx.positions,
            ctx.slot_of_token, cache.block_table, cache.k_pages, cache.v_pages, H, G, hd, cache.page_tokens,
            write_kv=write_cache, bias=self.b_qkv, pairing=pairing)
        att = torch.empty_like(q)
        ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.slot_of_token,
                            att, H, G, hd, cache.page_tokens, self.window or 0, self.scale,
                            plan=plan)
        ops.gemm(att, self.w_o, residual, accumulate=True, bias=self.b_o)


register_part("mixer", "gqa_attention", GQAAttention)

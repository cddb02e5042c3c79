"""Choice among the bfloat16 tensor-core matrix products.

  * up to 8 rows (small decode batches): the persistent TMA-ring streaming kernel (`gemm_stream.cu`) for large
    weights (gate/up, down, the output head), the weight-streaming mma.sync kernel (`gemm_smallm.cu`) for the
    smaller ones (q/k/v, o);
  * 9 to 16 rows: the streaming kernel at every shape;
  * more rows (larger decode batches, prefill, mixed batches): the persistent tcgen05 kernel (`gemm_tc.cu`) with
    the tile width that fills whole waves of SMs (`tc_config`), cutting K into slices when the output has fewer
    tiles than the GPU has SMs.
The choice depends on the shape alone, so a token's logits do not depend on what else a process ran before.
Shapes all of them refuse (K not a multiple of 8, unaligned operands) go to the generic kernel.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_UNSUPPORTED = 100001
SMALL_M = 64          # the most rows the weight-streaming kernel takes
SMALL_M_AUTO = 8      # up to here it is chosen (measured); above, the tcgen05 kernel with K slices streams better
_status = {}
_sm_count = {}


def status_flag(device: torch.device) -> torch.Tensor:
    """Device int32 that a timed-out wait inside a tensor-core kernel sets to 1."""
    key = device.index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device: torch.device) -> None:
    """Raises if a kernel recorded a timed-out wait (synchronises with the device)."""
    key = device.index or 0
    if key in _status and int(_status[key].item()) != 0:
        _status[key].zero_()
        raise RuntimeError("a tensor-core kernel gave up waiting on a barrier; its results are invalid")


def _sms(device: torch.device) -> int:
    key = device.index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _aligned(a, w) -> bool:
    return a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


_rt_override = 0      # tests and tuning runs may pin the row tiles per CTA


def row_tiles(M: int, N: int, device) -> int:
    """Row tiles of 16 per CTA for the small-M kernel.  One: measured fastest at every decode shape of the
    8B model (more, smaller CTAs per SM hide the latency of the weight loads better than fat ones)."""
    return _rt_override or 1


_tc_bn = 0            # tests and tuning runs may pin the tile width (a multiple of 16 up to 256) ...
_tc_splits = 0        # ... and the number of K slices of the tcgen05 kernel
TC_TILE_FIXED = 150   # a tile's fixed cost in columns: tiles of 128 measured 30-45 % slower per flop than tiles of 256


def tc_config(M: int, N: int, K: int, sms: int, swiglu: bool = False):
    """Tile width (a multiple of 16, of 32 with the SwiGLU epilogue) and number of K slices for the tcgen05 kernel.
    Many rows (prefill): the width, from 256 down to 192, whose tiles leave the least of the last wave of SMs
    empty, a tile costing its width plus a fixed part.  Few output tiles (decode batches, narrow outputs):
    with the SwiGLU epilogue the widest tile that gives every SM one (no slices: the epilogue cannot run on partial
    sums without a second kernel); else 128- or 256-wide tiles with K cut into slices so that every SM streams a
    share of the weights.  (A finer cost model that also weighed wave tails chose more slices and measured slower:
    the second kernel that adds the slices has a fixed cost.)"""
    m_tiles = -(-M // 128)
    step = 32 if swiglu else 16
    k_blocks = -(-K // 64)
    if _tc_bn:
        bn = _tc_bn
    elif m_tiles * -(-N // 256) >= sms:
        best = None
        for cand in range(256, 191, -step):
            waves = -(-(m_tiles * -(-N // cand)) // sms)
            cost = waves * (cand + TC_TILE_FIXED)
            if best is None or cost < best[0]:
                best = (cost, cand)
        bn = best[1]
    elif swiglu and m_tiles == 1:
        bn = min(256, max(32, -(-N // sms + step - 1) // step * step))       # the narrowest tile width that needs one wave
        while bn < 256 and -(-N // bn) > sms:
            bn += step
    else:
        bn = 256 if N >= 256 and m_tiles * -(-N // 256) >= sms // 2 else 128
    tiles = m_tiles * -(-N // bn)
    splits = 1
    if tiles < sms and not (swiglu and (N // 2) % (bn // 2)):
        splits = max(1, min(sms // tiles, k_blocks // 8))
    if _tc_splits:
        splits = min(_tc_splits, k_blocks)
    return bn, splits


STREAM_M = 32         # the most rows the persistent streaming kernel takes
STREAM_M_AUTO = 8     # up to here it is chosen ...
STREAM_MIN_WEIGHTS = 40 << 20    # ... for weights of at least this many elements (see `stream_wanted`)
STREAM_M_AUTO_WIDE = 16          # ... and up to here for weights of any size
_stream_rw = 0        # tests and tuning runs may pin the consumer warps across a tile's rows (8, 4, 2, 1)
_stream_ctas = 0      # tests may run fewer CTAs than SMs to move the places where CTAs hand a tile over
_stream_scratch = {}


STREAM_MAX_N = 1 << 20


def _stream_buffers(device: torch.device, lib):
    """Workspace for partial tiles and the per-tile arrival counters of the streaming kernel, sized once for
    the largest call it takes and never replaced (captured graphs keep their addresses).  One pair per device:
    the engine launches on one stream, and launches that do not overlap may share them."""
    key = device.index or 0
    if key not in _stream_scratch:
        if torch.cuda.is_current_stream_capturing():
            return None
        lib.hk_gemm_stream_workspace.restype = ctypes.c_longlong
        ws = torch.empty(int(lib.hk_gemm_stream_workspace(STREAM_M, 8)), dtype=torch.float32, device=device)
        ct = torch.zeros(STREAM_MAX_N // 16 + 2, dtype=torch.int32, device=device)
        _stream_scratch[key] = (ws, ct)
    return _stream_scratch[key]


def stream_row_warps(N: int, sms: int) -> int:
    """Consumer warps across a tile's rows (tile = 16 rows each): the widest tile that still gives every CTA a
    whole tile of its own, so that only the left-over tiles are shared between CTAs."""
    if _stream_rw:
        return _stream_rw
    for rw in (4, 2):
        if -(-N // (16 * rw)) >= sms:
            return rw
    return 1


def stream_wanted(M: int, N: int, K: int) -> bool:
    """The streaming kernel pays about two microseconds to fill its ring and to hand shared tiles over.  Measured
    on the 8B model's decode products: up to 8 rows it wins from about 80 MB of weights up (gate/up, down, output
    head) and loses to the small-M kernel below (q/k/v, o); from 9 to 16 rows it wins at every shape, against the
    small-M kernel and against the tcgen05 kernel with K slices; from 17 rows on the tcgen05 kernel is ahead."""
    if K % 64:
        return False
    return (M <= STREAM_M_AUTO and N * K >= STREAM_MIN_WEIGHTS) or STREAM_M_AUTO < M <= STREAM_M_AUTO_WIDE


def run_stream(a, w, out, epilogue: int, ldo: int) -> bool:
    """The persistent streaming kernel; epilogue 0 store, 1 add, 2 silu(gate) * up over w = [gate rows | up rows]."""
    from . import ops
    M, K = a.shape
    N = w.shape[0]
    if M > STREAM_M or N > STREAM_MAX_N:
        return False
    lib = build.load("gemm_stream")
    scratch = _stream_buffers(a.device, lib)
    if scratch is None:
        return False
    ws, ct = scratch
    code = lib.hk_gemm_stream(_ptr(a), _ptr(w), _ptr(out), M, N, K, ctypes.c_longlong(ldo), epilogue,
                              stream_row_warps(N, _sms(a.device)),
                              _ptr(ws), _ptr(ct), _ptr(status_flag(a.device)), _stream_ctas, _stream())
    if code == _UNSUPPORTED:
        return False
    ops._check(code, "gemm (streaming)")
    return True


def _tc_partial(lib, M: int, N: int, splits: int, device):
    """Scratch for the partial sums of `splits` K slices (None without slices)."""
    if splits <= 1:
        return None
    lib.hk_gemm_tc_partial_floats.restype = ctypes.c_longlong
    return torch.empty(int(lib.hk_gemm_tc_partial_floats(M, N, splits)), dtype=torch.float32, device=device)


def run(a, w, out, accumulate: bool, choice: Optional[str]) -> bool:
    """out (fp32) = a w^T (+ out).  Returns False when no tensor-core kernel takes the shape."""
    from . import ops
    M, K = a.shape
    N = w.shape[0]
    if not _aligned(a, w):
        return False
    if choice == "stream" or (choice is None and stream_wanted(M, N, K)):
        if run_stream(a, w, out, 1 if accumulate else 0, N):
            return True
        if choice == "stream":
            return False
    if choice == "smallm" or (choice is None and M <= SMALL_M_AUTO):
        if M > SMALL_M:
            return False
        lib = build.load("gemm_smallm")
        code = lib.hk_gemm_smallm(_ptr(a), _ptr(w), _ptr(out), M, N, K, ctypes.c_longlong(N), 1 if accumulate else 0,
                                  row_tiles(M, N, a.device), _stream())
        if code == _UNSUPPORTED:
            return False
        ops._check(code, "gemm (small-M)")
        return True
    lib = build.load("gemm_tc")
    bn, splits = tc_config(M, N, K, _sms(a.device))
    partial = _tc_partial(lib, M, N, splits, a.device)
    code = lib.hk_gemm_tc(_ptr(a), _ptr(w), _ptr(out), M, N, K, ctypes.c_longlong(N), 1 if accumulate else 0, bn,
                          splits, _ptr(partial) if splits > 1 else ctypes.c_void_p(0), _ptr(status_flag(a.device)), _stream())
    if code == _UNSUPPORTED:
        return False
    ops._check(code, "gemm (tcgen05)")
    return True


def run_swiglu(a, w_gate_up, out, choice: Optional[str] = None) -> bool:
    """out (bf16 [M, F]) = silu(gate) * up of a w^T for w = [F gate rows | F up rows], in the epilogue of the
    streaming kernel (few rows) or of the tcgen05 kernel; False when they refuse."""
    from . import ops
    M, K = a.shape
    N = w_gate_up.shape[0]
    if not _aligned(a, w_gate_up) or N % 2:
        return False
    if choice == "stream" or (choice is None and stream_wanted(M, N, K)):
        if N % (16 * stream_row_warps(N, _sms(a.device))) == 0 and run_stream(a, w_gate_up, out, 2, out.shape[1]):
            return True
        if choice == "stream":
            return False
    if choice is None and M <= SMALL_M_AUTO:
        return False             # few rows, small weights: the small-M product and the swiglu kernel
    lib = build.load("gemm_tc")
    bn, splits = tc_config(M, N, K, _sms(a.device), swiglu=True)
    partial = _tc_partial(lib, M, N, splits, a.device)
    code = lib.hk_gemm_tc(_ptr(a), _ptr(w_gate_up), _ptr(out), M, N, K, ctypes.c_longlong(out.shape[1]), 2, bn,
                          splits, _ptr(partial) if splits > 1 else ctypes.c_void_p(0), _ptr(status_flag(a.device)), _stream())
    if code == _UNSUPPORTED:
        return False
    ops._check(code, "gemm+swiglu (tcgen05)")
    return True

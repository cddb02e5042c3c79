"""Weights by tensor name: from a model folder's safetensors, or seeded random values.

The model's parts declare every tensor they need (name, shape, kind); this module knows
nothing else about a model.  Loading compares the declared set with the files' and reports
everything wrong in ONE error: missing tensors, unexpected tensors and wrong shapes, each
by name (the reference names the tensor and the expected shape the same way and refuses
unknown tensors rather than dropping them: src/engine/weights.zig:172-245,
src/convert/hf.zig:495-498).  Working types: matrices in the compute type (bfloat16, or
float32 on the true 32-bit path), vectors in float32, integer tables in int32.
`rotary_emb.inv_freq` buffers are skipped, as the reference's converter drops them
(src/convert/hf.zig:99,127).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..parts.base import ParamSpec, Precision, TABLE, VECTOR
from .safetensors_io import SafetensorsError, open_model_files, save_file

_FLOAT_DTYPES = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_INT_DTYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """Tensors of a model folder do not fit the model; `.missing`, `.unexpected`,
    `.wrong_shape` ({name: (found, expected)}) and `.wrong_dtype` hold the names."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = sorted(missing), sorted(unexpected)
        self.wrong_shape, self.wrong_dtype = dict(wrong_shape), dict(wrong_dtype)
        lines = [f"the tensors in '{where}' do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name in sorted(self.wrong_shape):
            found, want = self.wrong_shape[name]
            lines.append(f"  wrong shape: {name} is {list(found)}, expected {list(want)}")
        for name in sorted(self.wrong_dtype):
            lines.append(f"  wrong type: {name} is {self.wrong_dtype[name]}")
        super().__init__("\n".join(lines))


def _skipped(name: str) -> bool:
    return name.endswith("rotary_emb.inv_freq")


def load_tensors(model_dir: str, specs: Dict[str, ParamSpec], precision: Precision) -> Dict[str, torch.Tensor]:
    """Reads the declared tensors from `model_dir` to the device in their working types."""
    files = open_model_files(model_dir)
    where: Dict[str, object] = {}
    for f in files:
        for name in f.names():
            if not _skipped(name):
                where[name] = f
    missing = [n for n, s in specs.items() if n not in where and not s.optional]
    unexpected = [n for n in where if n not in specs]
    wrong_shape, wrong_dtype = {}, {}
    for name, spec in specs.items():
        if name not in where:
            continue
        dt, shape, _, _ = where[name].entries[name]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape[name] = (tuple(shape), tuple(spec.shape))
        tdt = where[name].tensor(name).dtype if tuple(shape) == tuple(spec.shape) else None
        if tdt is not None:
            ok = tdt in _INT_DTYPES if spec.kind == TABLE else tdt in _FLOAT_DTYPES
            if not ok:
                wrong_dtype[name] = f"{dt}, which a {spec.kind} cannot be read from"
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        if name in where:
            t = where[name].tensor(name)
            dtype = precision.working_dtype(spec.kind)
            if t.dtype == torch.float32 and dtype == torch.bfloat16:
                dtype = torch.float32          # a tensor stored in 32-bit stays so: the file says it needs them
            out[name] = t.to(device=precision.device, dtype=dtype).contiguous()
    for f in files:
        f.close()
    return out


def random_tensors(specs: Dict[str, ParamSpec], seed: int, std: float, norm_std: float,
                   device, dtype_of=None) -> Dict[str, torch.Tensor]:
    """Seeded random values for every declared, non-optional tensor: matrices N(0, std),
    norm-like vectors 1 + N(0, norm_std).  Each tensor has a stream of its own, derived from
    (seed, name), so the values do not depend on the order or on which other tensors exist, and
    the stream is counter-based with fixed arithmetic (`random_stream`), so they do not depend on
    the device either: a CUDA device fills the tensors with a kernel, the CPU with numpy, and
    both hold the same bits.  Values are made in float32 and cast to `dtype_of(spec)`
    (default float32)."""
    from . import random_stream
    device = torch.device(device)
    out = {}
    for name, spec in specs.items():
        if spec.optional:
            continue
        if spec.kind == TABLE:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        dtype = dtype_of(spec) if dtype_of is not None else torch.float32
        key = random_stream.tensor_key(seed, name)
        count = 1
        for n in spec.shape:
            count *= int(n)
        one_plus = spec.init == "one_plus_normal"
        scale, offset = (norm_std, 1.0) if one_plus else (std, 0.0)
        if device.type == "cuda" and dtype in (torch.float32, torch.bfloat16):
            import ctypes

            from ..csrc import build
            lib = build.load("random_init")
            t = torch.empty(spec.shape, dtype=dtype, device=device)
            with torch.cuda.device(device):
                code = lib.hk_random_init(ctypes.c_void_p(t.data_ptr()), 0 if dtype == torch.float32 else 1,
                                          ctypes.c_longlong(count), ctypes.c_ulonglong(key), ctypes.c_float(scale),
                                          ctypes.c_float(offset), 1 if one_plus else 0,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            if code != 0:
                raise RuntimeError(f"random_init: CUDA error {code}")
            out[name] = t
        else:
            host = torch.from_numpy(random_stream.fill(key, count, scale, offset)).reshape(spec.shape)
            out[name] = host.to(dtype).to(device)
    return out


def write_random_model(model_dir: str, config, seed: int, std: Optional[float] = None,
                       norm_std: float = 0.05, dtype: torch.dtype = torch.bfloat16) -> None:
    """Writes a model folder (config.json, model.safetensors) with seeded random weights of
    `config`'s architecture.  `std` defaults to the configuration's `initializer_range`.  Matrices are stored
    as `dtype`; vectors (norm weights) in float32, the type every engine computes them in, so that an engine that
    loads the folder and an engine given the same seed hold the same values."""
    from ..config import resolve_architecture
    _, build_model = resolve_architecture(config.architecture)
    spec = build_model(config, 8)
    if std is None:
        std = float(getattr(config, "initializer_range", 0.02))
    # the same bits on either device; a GPU, where there is one, fills large models in seconds
    device = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = random_tensors(spec.param_specs(), seed, std, norm_std, device,
                             dtype_of=lambda s: {TABLE: torch.int32, VECTOR: torch.float32}.get(s.kind, dtype))
    tensors = {k: v.cpu() for k, v in tensors.items()}
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    save_file(tensors, os.path.join(model_dir, "model.safetensors"))


__all__ = ["SafetensorsError", "WeightError", "load_tensors", "random_tensors", "write_random_model"]

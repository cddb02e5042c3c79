"""Reading and writing of safetensors files, by tensor name.

The format: an unsigned 64-bit little-endian header length, a JSON header
`{name: {dtype, shape, data_offsets}}` (the `__metadata__` entry is skipped), then the
tensors' bytes (the reference parses the same header: src/convert/hf.zig:403-479).  Files
are memory-mapped; a tensor is a view until it is copied to the device.  A sharded model
is followed through `model.safetensors.index.json`.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file; `entries` maps a tensor name to (dtype name, shape, begin, end)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}'") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            count = 1
            for s in shape:
                count *= s
            if e - b != count * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' holds {e - b} bytes but shape {list(shape)} of {dt} needs {count * _DTYPES[dt][1]}")
            if b < 0 or self._base + e > size:
                raise SafetensorsError(f"{path}: tensor '{name}' lies outside the file")
            self.entries[name] = (dt, shape, int(b), int(e))

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only memory: copy before writing)."""
        dt, shape, b, e = self.entries[name]
        tdt, _ = _DTYPES[dt]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._base + b:self._base + e]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # "buffer is not writable": it is only read
            flat = torch.frombuffer(buf, dtype=torch.uint8)
        return flat.view(tdt).reshape(shape)

    def close(self) -> None:
        # Views may still reference the map; the OS drops it when they go.
        self._f.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The safetensors files of a model folder: the index's shards, else model.safetensors,
    else every *.safetensors in name order."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted(set(wm.values()))
    elif os.path.isfile(os.path.join(model_dir, "model.safetensors")):
        files = ["model.safetensors"]
    else:
        files = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no safetensors file in '{model_dir}'")
    return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in files]


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    """Writes `tensors` (CPU or device) as one safetensors file, names in sorted order."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)

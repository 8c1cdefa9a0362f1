"""Reader and writer for the safetensors container.

Layout: an unsigned 64-bit little-endian header length, a JSON header mapping each
tensor name to {dtype, shape, data_offsets}, then the raw little-endian tensor bytes.
The reference reads GGUF only (crates/gguf/src/parse.rs:53-65); this is the same job
for the other container: a read-only memory map, tensors looked up by name, every
offset checked against the file before it is used, errors instead of crashes.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict

import numpy as np
import torch

from ..errors import FileFormatError

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` returns a CPU view (no copy)."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise FileFormatError(f"cannot open {path}: {e}") from None
        size = self._fh.seek(0, 2)
        self._fh.seek(0)
        if size < 8:
            raise FileFormatError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > MAX_HEADER or 8 + n > size:
            raise FileFormatError(f"{path}: header length {n} exceeds the file")
        try:
            header = json.loads(self._fh.read(n))
        except ValueError as e:
            raise FileFormatError(f"{path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise FileFormatError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data0 = 8 + n
        data_len = size - self._data0
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self.entries: Dict[str, dict] = {}
        for name, info in header.items():
            try:
                dt, shape, (lo, hi) = info["dtype"], list(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise FileFormatError(f"{path}: malformed entry for tensor {name}") from None
            if dt not in _DTYPES:
                raise FileFormatError(f"{path}: tensor {name} has unsupported dtype {dt}")
            count = 1
            for s in shape:
                if not isinstance(s, int) or s < 0:
                    raise FileFormatError(f"{path}: tensor {name} has a bad shape {shape}")
                count *= s
            if not (isinstance(lo, int) and isinstance(hi, int) and 0 <= lo <= hi <= data_len):
                raise FileFormatError(f"{path}: tensor {name} lies outside the file")
            if hi - lo != count * _DTYPES[dt][1]:
                raise FileFormatError(f"{path}: tensor {name}: {hi - lo} bytes for shape {shape} of {dt}")
            self.entries[name] = {"dtype": dt, "shape": shape, "lo": lo, "hi": hi}

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return tuple(self.entries[name]["shape"])

    def dtype(self, name) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name) -> torch.Tensor:
        e = self.entries[name]
        tdt, size = _DTYPES[e["dtype"]]
        count = (e["hi"] - e["lo"]) // size
        if count == 0:
            return torch.empty(e["shape"], dtype=tdt)
        buf = memoryview(self._map)[self._data0 + e["lo"]: self._data0 + e["hi"]]
        # a read-only map: torch warns about non-writable buffers, the view is never written
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=tdt, count=count)
        return t.reshape(e["shape"])

    def close(self):
        self._map = None
        self._fh.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    """Write name -> tensor (CPU, contiguous) in name order, data 8-byte aligned."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise FileFormatError(f"cannot store dtype {t.dtype} of {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for raw in blobs:
            f.write(raw)

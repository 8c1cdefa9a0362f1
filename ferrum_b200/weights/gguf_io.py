"""Reader and writer for unquantized GGUF files (F32, F16, BF16 tensors).

Format, versions 2 and 3: magic "GGUF", u32 version, u64 tensor count, u64 key-value count,
the key-value pairs, the tensor directory (name, dims innermost first, ggml type, offset),
zero padding to `general.alignment` (default 32), tensor data.  The checks are the
reference's (crates/gguf/src/parse.rs:99-173, :304-346): bad magic or version, counts that
exceed the bytes left, alignment that is not a non-zero multiple of 8, non-zero padding,
unaligned or out-of-file tensor data, duplicate names, arrays nested deeper than 64,
booleans other than 0/1, strings that are not UTF-8 are errors, never crashes.  Quantized
ggml types are named in the error and refused (quantization is not part of this engine).
"""
from __future__ import annotations

import mmap
import struct
from typing import Dict, List

import torch

from ..errors import FileFormatError

MAGIC = b"GGUF"
MAX_ARRAY_DEPTH = 64
# ggml type id -> (name, torch dtype or None, block elements, block bytes); crates/gguf/src/layout.rs:12-45
GGML_TYPES = {0: ("F32", torch.float32, 1, 4), 1: ("F16", torch.float16, 1, 2), 30: ("BF16", torch.bfloat16, 1, 2),
              2: ("Q4_0", None, 32, 18), 3: ("Q4_1", None, 32, 20), 6: ("Q5_0", None, 32, 22), 7: ("Q5_1", None, 32, 24),
              8: ("Q8_0", None, 32, 34), 9: ("Q8_1", None, 32, 36), 10: ("Q2_K", None, 256, 84),
              11: ("Q3_K", None, 256, 110), 12: ("Q4_K", None, 256, 144), 13: ("Q5_K", None, 256, 176),
              14: ("Q6_K", None, 256, 210), 15: ("Q8_K", None, 256, 292), 24: ("I8", None, 1, 1), 25: ("I16", None, 1, 2),
              26: ("I32", None, 1, 4), 27: ("I64", None, 1, 8), 28: ("F64", None, 1, 8)}
_TORCH_TO_GGML = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}
T_BOOL, T_STRING, T_ARRAY = 7, 8, 9


class _Reader:
    def __init__(self, data):
        self.data, self.pos = data, 0

    def take(self, n):
        if n < 0 or self.pos + n > len(self.data):
            raise FileFormatError("gguf: unexpected end of file")
        b = self.data[self.pos:self.pos + n]
        self.pos += n
        return b

    def scalar(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def remaining(self):
        return len(self.data) - self.pos

    def count(self, min_elem):
        """A u64 count that the bytes left can actually hold (crates/gguf/src/parse.rs:338-346)."""
        n = self.scalar("<Q")
        if n > self.remaining() // max(1, min_elem):
            raise FileFormatError("gguf: count exceeds remaining bytes")
        return n

    def string(self):
        n = self.count(1)
        try:
            return bytes(self.take(n)).decode("utf-8")
        except UnicodeDecodeError:
            raise FileFormatError("gguf: string is not valid UTF-8") from None

    def value(self, vtype, depth=0):
        if vtype in _SCALARS:
            return self.scalar(_SCALARS[vtype])
        if vtype == T_BOOL:
            b = self.scalar("<B")
            if b > 1:
                raise FileFormatError("gguf: bool is not 0 or 1")
            return bool(b)
        if vtype == T_STRING:
            return self.string()
        if vtype == T_ARRAY:
            if depth >= MAX_ARRAY_DEPTH:
                raise FileFormatError("gguf: arrays nested too deeply")
            etype = self.scalar("<I")
            size = struct.calcsize(_SCALARS[etype]) if etype in _SCALARS else (1 if etype == T_BOOL else 8)
            if etype not in _SCALARS and etype not in (T_BOOL, T_STRING, T_ARRAY):
                raise FileFormatError(f"gguf: unknown metadata type {etype}")
            n = self.count(size if etype != T_ARRAY else 12)
            return [self.value(etype, depth + 1) for _ in range(n)]
        raise FileFormatError(f"gguf: unknown metadata type {vtype}")


class GGUFFile:
    """A memory-mapped GGUF file: `metadata` (dict) and tensors by name (CPU views)."""

    def __init__(self, path):
        self.path = path
        try:
            self._fh = open(path, "rb")
            size = self._fh.seek(0, 2)
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else b""
        except (OSError, ValueError) as e:
            raise FileFormatError(f"cannot open {path}: {e}") from None
        r = _Reader(memoryview(self._map))
        if bytes(r.take(4)) != MAGIC:
            raise FileFormatError("gguf: bad gguf magic")
        self.version = r.scalar("<I")
        if self.version not in (2, 3):
            raise FileFormatError(f"gguf: unsupported gguf version {self.version}")
        n_tensors = r.count(1)
        n_kv = r.count(1)
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = r.string()
            if key in self.metadata:
                raise FileFormatError(f"gguf: duplicate metadata key {key}")
            self.metadata[key] = r.value(r.scalar("<I"))
        self.alignment = self.metadata.get("general.alignment", 32)
        if not isinstance(self.alignment, int) or isinstance(self.alignment, bool) or self.alignment <= 0 or self.alignment % 8:
            raise FileFormatError("gguf: alignment must be a non-zero multiple of 8")
        raw = []
        for _ in range(n_tensors):
            name = r.string()
            nd = r.scalar("<I")
            if nd > 8:
                raise FileFormatError(f"gguf: tensor {name} has {nd} dimensions")
            dims = [r.scalar("<Q") for _ in range(nd)]
            gtype = r.scalar("<I")
            offset = r.scalar("<Q")
            raw.append((name, dims, gtype, offset))
        data_start = r.pos + (-r.pos) % self.alignment
        if data_start > len(r.data):
            if raw:
                raise FileFormatError("gguf: alignment padding exceeds file")
            data_start = len(r.data)
        if any(bytes(r.data[r.pos:data_start])):
            raise FileFormatError("gguf: alignment padding is not zero")
        self._data0 = data_start
        data_len = len(r.data) - data_start
        self.entries: Dict[str, dict] = {}
        self.order: List[str] = []
        for name, dims, gtype, offset in raw:
            if name in self.entries:
                raise FileFormatError(f"gguf: duplicate tensor {name}")
            if gtype not in GGML_TYPES:
                raise FileFormatError(f"gguf: tensor {name} has unknown ggml type {gtype}")
            tname, tdt, block, bbytes = GGML_TYPES[gtype]
            count = 1
            for d in dims:
                count *= d
                if count > (1 << 62):
                    raise FileFormatError(f"gguf: tensor {name} size overflows")
            if dims and block > 1 and dims[0] % block:
                raise FileFormatError(f"gguf: tensor {name} row length is not a multiple of its block size")
            nbytes = count // block * bbytes
            if offset % self.alignment:
                raise FileFormatError(f"gguf: tensor {name} data_offset is not aligned")
            if offset + nbytes > data_len:
                raise FileFormatError(f"gguf: tensor {name} extends past end of file")
            self.entries[name] = {"dims": dims, "type": gtype, "offset": offset, "nbytes": nbytes}
            self.order.append(name)

    def names(self):
        return list(self.order)

    def shape(self, name):
        """Row-major shape: GGUF lists the innermost dimension first."""
        return tuple(reversed(self.entries[name]["dims"]))

    def dtype(self, name):
        return GGML_TYPES[self.entries[name]["type"]][1]

    def type_name(self, name):
        return GGML_TYPES[self.entries[name]["type"]][0]

    def tensor(self, name) -> torch.Tensor:
        e = self.entries[name]
        tname, tdt, _, _ = GGML_TYPES[e["type"]]
        if tdt is None:
            raise FileFormatError(f"gguf: tensor {name} has type {tname}; only F32, F16 and BF16 are computable here")
        shape = self.shape(name)
        if e["nbytes"] == 0:
            return torch.empty(shape, dtype=tdt)
        import warnings
        buf = memoryview(self._map)[self._data0 + e["offset"]: self._data0 + e["offset"] + e["nbytes"]]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=tdt, count=e["nbytes"] // tdt.itemsize)
        return t.reshape(shape)

    def dump(self) -> str:
        """The reference's listing (crates/core-types/src/source.rs:71-92): a header, then one
        tensor per line in file order, dims innermost first."""
        out = [f"ferrum-gguf version={self.version} alignment={self.alignment} metadata={len(self.metadata)} "
               f"tensors={len(self.order)}"]
        for n in self.order:
            e = self.entries[n]
            out.append(f"{n} [{', '.join(str(d) for d in e['dims'])}] {GGML_TYPES[e['type']][0]}")
        return "\n".join(out) + "\n"


def _pack_string(s):
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _pack_value(v):
    """(type id, bytes).  ints become u32 when they fit, else u64/i64; floats f32."""
    if isinstance(v, bool):
        return T_BOOL, struct.pack("<B", int(v))
    if isinstance(v, int):
        if 0 <= v < 2 ** 32:
            return 4, struct.pack("<I", v)
        return (10, struct.pack("<Q", v)) if v >= 0 else (11, struct.pack("<q", v))
    if isinstance(v, float):
        return 6, struct.pack("<f", v)
    if isinstance(v, str):
        return T_STRING, _pack_string(v)
    if isinstance(v, (list, tuple)):
        if not v:
            return T_ARRAY, struct.pack("<IQ", 4, 0)
        packed = [_pack_value(x) for x in v]
        etype = packed[0][0]
        if any(p[0] != etype for p in packed):
            raise FileFormatError("gguf: array elements must share a type")
        return T_ARRAY, struct.pack("<IQ", etype, len(v)) + b"".join(p[1] for p in packed)
    raise FileFormatError(f"gguf: cannot store metadata value of type {type(v).__name__}")


def write_gguf(path, metadata: Dict[str, object], tensors: Dict[str, torch.Tensor], alignment=32, version=3):
    """Write a v3 file with the tensors in the given order (F32, F16 or BF16)."""
    meta = dict(metadata)
    if alignment != 32:
        meta["general.alignment"] = int(alignment)
    head = MAGIC + struct.pack("<IQQ", version, len(tensors), len(meta))
    for k, v in meta.items():
        t, b = _pack_value(v)
        head += _pack_string(k) + struct.pack("<I", t) + b
    offset, infos, blobs = 0, b"", []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _TORCH_TO_GGML:
            raise FileFormatError(f"gguf: cannot store dtype {t.dtype} of {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        dims = list(reversed(t.shape))
        infos += _pack_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", _TORCH_TO_GGML[t.dtype], offset)
        pad = (-len(raw)) % alignment
        blobs.append(raw + b"\0" * pad)
        offset += len(raw) + pad
    head += infos
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)

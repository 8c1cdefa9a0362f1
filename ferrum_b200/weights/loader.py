"""Loads a model's weights by tensor name, with one error that lists everything wrong.

The reference validates a closed set of names: any tensor it does not expect, any bias, any
wrong shape or uncomputable dtype is a load error (crates/model/src/weights.rs:157-230), and
a missing `output.weight` means the output shares the embedding (crates/model/src/llama.rs:
103-111).  Same rules here, except that all problems are collected into a single
`WeightsError` instead of stopping at the first.

Storage policy: matrices are kept in the compute dtype (bfloat16, float16 or float32: a
float16 file computed in float16 is used as stored, as the reference does with F16 weights,
crates/core-types/src/dtype.rs:24-45; float16 and bfloat16 files upcast exactly for the
float32 path; a file of the other 16-bit type is rounded), vectors such as norm weights stay
float32, integer tables become int32.
"""
from __future__ import annotations

import glob
import os

import torch

from ..errors import FileFormatError, WeightsError
from .safetensors_io import SafetensorsFile

_KIND_DTYPE = {"vector": torch.float32, "table": torch.int32}


class _Source:
    """name -> (shape, loader) over one or more files."""

    def __init__(self):
        self.entries = {}

    def add(self, name, shape, dtype, fetch):
        if name in self.entries:
            raise FileFormatError(f"tensor {name} appears twice")
        self.entries[name] = (tuple(shape), dtype, fetch)


def open_source(path):
    """A model folder (every *.safetensors in it) or a single .safetensors / .gguf file."""
    src = _Source()
    if os.path.isdir(path):
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
        if not files:
            raise FileFormatError(f"{path}: no .safetensors file")
    else:
        files = [path]
    for f in files:
        if f.endswith(".gguf"):
            from .gguf_io import GGUFFile
            g = GGUFFile(f)
            for name in g.names():
                src.add(name, g.shape(name), g.dtype(name), (lambda n=name, g=g: g.tensor(n)))
        else:
            st = SafetensorsFile(f)
            for name in st.names():
                src.add(name, st.shape(name), st.dtype(name), (lambda n=name, st=st: st.tensor(n)))
    return src


def check_weights(specs, available, rename=None):
    """Compare what the model wants with what the file has.

    specs: canonical name -> ParamSpec; available: file name -> shape; rename: file name ->
    canonical name (names not in it keep their own).  Returns canonical -> file name, or
    raises one WeightsError listing missing, unexpected and misshapen tensors.
    """
    rename = rename or {}
    found, unexpected, wrong = {}, [], []
    for fname, shape in available.items():
        canon = rename.get(fname, fname)
        if canon not in specs:
            unexpected.append(fname)
            continue
        found[canon] = fname
        want = tuple(specs[canon].shape)
        if tuple(shape) != want:
            wrong.append(f"{fname}: shape {list(shape)}, expected {list(want)}")
    missing = [n for n, s in specs.items() if n not in found and not s.optional]
    if missing or unexpected or wrong:
        back = {v: k for k, v in rename.items()}
        parts = []
        if missing:
            parts.append("missing: " + ", ".join(sorted(back.get(m, m) for m in missing)))
        if unexpected:
            parts.append("unexpected: " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append("wrong shape: " + "; ".join(sorted(wrong)))
        raise WeightsError("weights do not match the model -- " + " | ".join(parts))
    return found


def convert(t, kind, compute_dtype):
    want = _KIND_DTYPE.get(kind, compute_dtype)
    if kind == "matrix" and not t.dtype.is_floating_point:
        raise WeightsError(f"a matrix is stored as {t.dtype}")
    return t if t.dtype == want else t.to(want)


def load_weights(model, path, rename=None, device="cuda"):
    """Fill `model` (a tree of parts) from the files at `path` and finalize it."""
    src = open_source(path)
    specs = model.weight_specs()
    found = check_weights({n: s for n, (s, _, _) in specs.items()}, {n: e[0] for n, e in src.entries.items()}, rename)
    for canon, fname in found.items():
        spec, part, local = specs[canon]
        t = src.entries[fname][2]()
        part.assign(local, convert(t, spec.kind, model.dtype).to(device, non_blocking=False).contiguous())
    model.finalize()
    return model

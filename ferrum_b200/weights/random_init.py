"""Random-weights mode: fills a model, or writes a model folder, from a config and a seed.

Every tensor has its own generator keyed by (seed, name), so values do not depend on the
order or the set of tensors: matrices are N(0, 0.02), norm weights 1 + N(0, 0.02).  The
reference has no such mode (its tests fill every weight with 0.01,
crates/model/src/tests.rs:25-34).
"""
from __future__ import annotations

import json
import os
import zlib

import torch

from ..config import registry
from .loader import convert
from .safetensors_io import write_safetensors

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}

# How a parameter is drawn, by the `init` of its ParamSpec: a name registered here, or a function
# (shape, generator, device, std) -> float32 tensor given in the spec itself.  A part that needs
# another distribution brings it along; nothing here has to change.
INITS = {
    "normal": lambda shape, g, device, std: torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std,
    "ones_normal": lambda shape, g, device, std: 1.0 + torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std,
    "zeros": lambda shape, g, device, std: torch.zeros(shape, device=device, dtype=torch.float32),
}


def register_init(name, fn):
    INITS[name] = fn


def _tensor(name, spec, seed, device, std):
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    if spec.kind == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    draw = spec.init if callable(spec.init) else INITS.get(spec.init)
    if draw is None:
        raise ValueError(f"{name}: unknown initialisation {spec.init!r} (registered: {', '.join(sorted(INITS))})")
    return draw(tuple(spec.shape), g, device, std)


def init_random(model, seed, device="cuda", std=0.02):
    """Assign random values to every parameter of `model` on `device` and finalize it."""
    for name, (spec, part, local) in model.weight_specs().items():
        if spec.optional:
            continue          # e.g. an output matrix the model can share with the embedding
        part.assign(local, convert(_tensor(name, spec, seed, device, std), spec.kind, model.dtype).contiguous())
    model.finalize()
    return model


def write_random_model(config_dict, folder, seed, dtype="float32", std=0.02, tie=None):
    """Write `folder/config.json` and `folder/model.safetensors` for the architecture that
    config_dict names; tensor names are the checkpoint's (HF) names."""
    arch = registry.lookup(str(config_dict["architectures"][0]))
    cfg = arch.read_config(config_dict)
    model = arch.build(cfg, _DT[dtype], "cpu", max_positions=1)
    back = {v: k for k, v in (arch.hf_names(cfg) if arch.hf_names else {}).items()}
    tied = getattr(cfg, "tie_word_embeddings", False) if tie is None else tie
    tensors = {}
    for name, (spec, _, _) in model.weight_specs().items():
        if spec.optional and tied:
            continue
        t = _tensor(name, spec, seed, "cpu", std)
        store = _DT[dtype] if spec.kind == "matrix" else (torch.int32 if spec.kind == "table" else torch.float32)
        tensors[back.get(name, name)] = t.to(store)
    os.makedirs(folder, exist_ok=True)
    out = dict(config_dict)
    out["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
    return folder


def write_random_gguf(config_dict, path, seed, dtype="float16", std=0.02):
    """Write a GGUF file (canonical tensor names, metadata keys of the reference) with the same
    random values that `write_random_model` draws for this config and seed.  Rows of the q and
    k matrices are stored as drawn, so the file means "adjacent-pair rotation" as every GGUF
    Llama file does."""
    from .gguf_io import write_gguf
    store = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    arch = registry.lookup(str(config_dict["architectures"][0]))
    cfg = arch.read_config(config_dict)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=1)
    tied = getattr(cfg, "tie_word_embeddings", False)
    tensors = {}
    for name, (spec, _, _) in model.weight_specs().items():
        if spec.optional and tied:
            continue
        t = _tensor(name, spec, seed, "cpu", std)
        tensors[name] = t.to(store if spec.kind == "matrix" else torch.float32)
    write_gguf(path, cfg.to_gguf_metadata(), tensors)
    return path

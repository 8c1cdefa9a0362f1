"""One registry from an architecture's name to its configuration reader and its model.

The reference checks the architecture with a string compare inside its config reader
(crates/core-types/src/model.rs:65-70) and has one model.  Here the name found in
config.json (`architectures[0]`) or in GGUF metadata (`general.architecture`) selects
an entry; everything else in the package asks the registry and never names a model.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict

from ..errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[dict], object]      # config.json dict -> typed config
    build: Callable[..., object]               # (config, dtype, device) -> model (parts put together)
    hf_names: Callable[[object], Dict[str, str]] = None   # typed config -> {file tensor name: model tensor name}
    read_gguf: Callable[..., object] = None               # (opened GGUF file: .metadata, .entries, .shape(), .dtype()) -> typed config


_REGISTRY: Dict[str, Architecture] = {}


def register(arch: Architecture, *aliases: str) -> None:
    for key in (arch.name,) + aliases:
        _REGISTRY[key] = arch


def unregister(name: str) -> None:
    _REGISTRY.pop(name, None)


def lookup(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _REGISTRY[name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY)) or "none"
        raise ConfigError(f"unsupported architecture {name} (registered: {known})") from None


def names():
    _ensure_builtin()
    return sorted(_REGISTRY)


def read_config(folder_or_file: str):
    """(Architecture, typed config) of a model folder, a config.json path or a .gguf file."""
    path = folder_or_file
    if path.endswith(".gguf"):
        from ..weights.gguf_io import GGUFFile
        g = GGUFFile(path)
        arch = lookup(str(g.metadata.get("general.architecture")))
        if arch.read_gguf is None:
            raise ConfigError(f"architecture {arch.name} cannot be read from GGUF metadata")
        return arch, arch.read_gguf(g)
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            d = json.load(f)
    except (OSError, ValueError) as e:
        raise ConfigError(f"cannot read {path}: {e}") from None
    if not isinstance(d, dict) or not d.get("architectures"):
        raise ConfigError(f"{path}: no 'architectures' entry")
    arch = lookup(str(d["architectures"][0]))
    return arch, arch.read_config(d)


def _ensure_builtin():
    if "LlamaForCausalLM" not in _REGISTRY:
        from ..models import llama  # noqa: F401  (registers itself)

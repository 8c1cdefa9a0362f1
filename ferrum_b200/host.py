"""The native host module (C++ cache manager and scheduler), built at first use."""
from __future__ import annotations

import importlib
import threading

from .errors import KernelError
from .ops import build

_mod = None
_lock = threading.Lock()
ABI = 5


def module():
    global _mod
    if _mod is None:
        with _lock:
            if _mod is None:
                build.build_host()
                try:
                    m = importlib.import_module("ferrum_b200._host")
                except ImportError as e:
                    raise KernelError(f"cannot load the native host module: {e}") from None
                if getattr(m, "ABI", None) != ABI:
                    raise KernelError("the native host module is a stale build; delete ferrum_b200/_host*.so")
                _mod = m
    return _mod

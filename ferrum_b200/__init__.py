"""ferrum_b200: a single-GPU Llama inference engine for NVIDIA B200 (sm_100a).

Everything between a request's token ids and its next token: typed configuration and a
model registry, safetensors/GGUF weights, a model put together from parts, a paged cache
manager, one step function for mixed batches, a continuous batcher, samplers, and
hand-written CUDA kernels.
"""
__version__ = "0.2.0"
# Counts changes of what callers write against: the names and meanings of Engine's methods, of the
# command line's options and of the parts' interfaces (the reference freezes its own the same way:
# crates/core-types/src/lib.rs:45, tests/accept/tests/interface_revision.rs).  A test holds the
# surface that this number stands for.
INTERFACE_REVISION = 2

from .errors import (CacheError, ConfigError, FerrumError, FileFormatError, InvalidRequest, KernelError, NotFound,
                     SchedulerError, Unavailable, WeightsError)

__all__ = ["CacheError", "ConfigError", "FerrumError", "FileFormatError", "InvalidRequest", "KernelError", "NotFound",
           "SchedulerError", "Unavailable", "WeightsError", "Engine", "SamplingParams", "load_model", "INTERFACE_REVISION"]


def __getattr__(name):
    if name in ("Engine", "SamplingParams", "load_model"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)

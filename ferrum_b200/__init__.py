"""ferrum_b200: a single-GPU Llama inference engine for NVIDIA B200 (sm_100a).

Everything between a request's token ids and its next token: typed configuration and a
model registry, safetensors/GGUF weights, a model put together from parts, a paged cache
manager, one step function for mixed batches, a continuous batcher, samplers, and
hand-written CUDA kernels.
"""
__version__ = "0.1.0"

from .errors import (CacheError, ConfigError, FerrumError, FileFormatError, InvalidRequest, KernelError, NotFound,
                     SchedulerError, Unavailable, WeightsError)

__all__ = ["CacheError", "ConfigError", "FerrumError", "FileFormatError", "InvalidRequest", "KernelError", "NotFound",
           "SchedulerError", "Unavailable", "WeightsError", "Engine", "SamplingParams", "load_model"]


def __getattr__(name):
    if name in ("Engine", "SamplingParams", "load_model"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)

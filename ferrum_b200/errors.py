"""Error classes of the engine.

The variants follow the reference's error enum (crates/core-types/src/error.rs:22-46):
one class per place that can refuse: a request, a file, a weight set, a kernel, the
cache, the scheduler.  The HTTP mapping of the reference is not kept (no server here).
"""


class FerrumError(Exception):
    """Base of every error the engine raises on purpose."""


class InvalidRequest(FerrumError):
    """A request the engine will not run (empty prompt, id outside the vocabulary, ...)."""

    def __init__(self, message, param=None):
        super().__init__(message)
        self.param = param


class NotFound(FerrumError):
    """A request id that is neither queued nor running."""


class Unavailable(FerrumError):
    """No room right now (no request slot, no page); the caller may try again later."""


class ConfigError(FerrumError):
    """config.json or GGUF metadata that does not describe a model this engine builds."""


class FileFormatError(FerrumError):
    """A weight file that cannot be parsed (the reference's `Gguf` variant)."""


class WeightsError(FerrumError):
    """A weight set that does not match the model: missing, unexpected or misshapen
    tensors, all listed in one message (the reference's `Model` variant)."""


class KernelError(FerrumError):
    """A kernel refused its arguments, or the CUDA extension is missing."""


class CacheError(FerrumError):
    """Misuse of the cache manager: double free, unknown request, table too narrow."""


class SchedulerError(FerrumError):
    """An inconsistency inside the scheduler."""

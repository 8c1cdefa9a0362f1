from .llama import LlamaConfig, RopeScaling
from .registry import Architecture, register, unregister, lookup, names, read_config

__all__ = ["LlamaConfig", "RopeScaling", "Architecture", "register", "unregister", "lookup", "names",
           "read_config"]

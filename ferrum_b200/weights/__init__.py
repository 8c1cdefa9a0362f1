from .gguf_io import GGUFFile, write_gguf
from .loader import check_weights, load_weights, open_source
from .random_init import init_random, write_random_gguf, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["check_weights", "load_weights", "open_source", "init_random", "write_random_model", "write_random_gguf", "SafetensorsFile",
           "write_safetensors", "GGUFFile", "write_gguf"]

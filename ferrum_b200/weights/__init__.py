from .loader import check_weights, load_weights, open_source
from .random_init import init_random, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["check_weights", "load_weights", "open_source", "init_random", "write_random_model", "SafetensorsFile",
           "write_safetensors"]

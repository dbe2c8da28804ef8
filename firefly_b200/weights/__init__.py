from .loader import WeightError, WeightSpec, load_weights, storage_dtype
from .random_init import random_weights, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["WeightError", "WeightSpec", "load_weights", "storage_dtype", "random_weights",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "save_safetensors"]

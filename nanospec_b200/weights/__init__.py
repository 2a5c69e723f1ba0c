from .loader import WeightError, build_model, load_model, update_weights
from .random_init import random_model, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "build_model", "load_model", "random_model",
           "update_weights", "write_random_model", "write_safetensors"]

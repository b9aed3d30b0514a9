from .loader import WeightError, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, save_tensors, write_safetensors

__all__ = ["WeightError", "load_weights", "write_random_model", "random_tensors", "ModelFiles", "SafetensorsError",
           "SafetensorsFile", "save_tensors", "write_safetensors"]

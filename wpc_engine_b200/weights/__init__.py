from .loader import WeightError, bind_model, load_weights
from .random_init import random_weights_on_device, write_random_model
from .safetensors_io import ModelFiles, SafetensorsFile, WeightFileError, write_safetensors

__all__ = ["ModelFiles", "SafetensorsFile", "WeightError", "WeightFileError", "bind_model",
           "load_weights", "random_weights_on_device", "write_random_model", "write_safetensors"]

from .loader import WeightError, load_tensors, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "load_tensors", "random_tensor",
           "write_random_model", "write_safetensors"]

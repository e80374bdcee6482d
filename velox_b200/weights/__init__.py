from .loader import WeightError, load_weights
from .random_init import bind_random_weights, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, model_files, write_safetensors

__all__ = ["WeightError", "load_weights", "bind_random_weights", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "model_files", "write_safetensors"]

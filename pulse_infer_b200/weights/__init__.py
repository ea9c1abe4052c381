from .loader import WeightError, load_weights
from .random_init import init_random_weights, normal_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, list_weight_files, write_safetensors

__all__ = ["WeightError", "load_weights", "init_random_weights", "normal_tensor", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "list_weight_files", "write_safetensors"]

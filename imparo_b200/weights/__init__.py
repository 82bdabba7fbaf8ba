from .loader import WeightError, load_weights
from .random_init import write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["WeightError", "load_weights", "write_random_model", "SafetensorsFile", "write_safetensors"]

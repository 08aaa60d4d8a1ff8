from .errors import WeightError
from .safetensors_io import SafetensorsFile, save_file
from .loader import expected_tensors, load_weights
from .random_init import InitSpec, write_random_model

__all__ = ["WeightError", "SafetensorsFile", "save_file", "expected_tensors", "load_weights",
           "InitSpec", "write_random_model"]

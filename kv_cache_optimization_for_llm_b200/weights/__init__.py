from .loader import WeightError, WeightSpec, check_and_load, to_compute
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, read_header, read_tensors, write_tensors

__all__ = ["WeightError", "WeightSpec", "check_and_load", "to_compute", "random_tensors",
           "write_random_model", "SafetensorsError", "read_header", "read_tensors", "write_tensors"]

from .loader import INT_TABLE, MATRIX, VECTOR, TensorSpec, WeightError, check_index, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors import SafetensorsError, TensorEntry, index_folder, read_index, read_tensor, write_safetensors

__all__ = ["INT_TABLE", "MATRIX", "VECTOR", "TensorSpec", "WeightError", "check_index", "load_tensors",
           "random_tensors", "write_random_model", "SafetensorsError", "TensorEntry", "index_folder",
           "read_index", "read_tensor", "write_safetensors"]

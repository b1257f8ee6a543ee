from .loader import IGNORED_TENSORS, WeightError, check_against, load_tensors, storage_dtype
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["IGNORED_TENSORS", "WeightError", "check_against", "load_tensors", "storage_dtype",
           "random_tensor", "random_tensors", "write_random_model",
           "SafetensorsError", "SafetensorsFile", "open_model_files", "write_safetensors"]

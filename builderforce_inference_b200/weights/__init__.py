from .loader import WeightsError, load_folder
from .random_init import expected_tensors, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightsError", "load_folder", "expected_tensors", "random_tensors", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "write_safetensors"]

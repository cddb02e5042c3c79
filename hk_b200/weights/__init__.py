from .loader import WeightError, load_tensors, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_file

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightError", "load_tensors", "open_model_files",
           "random_tensors", "save_file", "write_random_model"]

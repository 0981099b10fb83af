from .loader import DEFAULT_IGNORED, WeightError, check_table, choose_prefix, folder_names, load_tensors, target_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, SafetensorsFolder, write_safetensors

__all__ = ["DEFAULT_IGNORED", "WeightError", "check_table", "choose_prefix", "folder_names", "load_tensors",
           "target_dtype", "random_tensors", "write_random_model", "SafetensorsError", "SafetensorsFile",
           "SafetensorsFolder", "write_safetensors"]

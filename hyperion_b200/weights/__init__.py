from .loader import WeightsError, check_tensors, load_weights
from .random_init import init_random, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, read_all, read_header, read_model_index, write_file

__all__ = ["WeightsError", "check_tensors", "load_weights", "init_random", "random_tensors", "write_model_folder",
           "SafetensorsError", "read_all", "read_header", "read_model_index", "write_file"]

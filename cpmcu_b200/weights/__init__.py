from .loader import WeightError, check_and_place, load_checkpoint
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, model_files, save_file

__all__ = ["WeightError", "check_and_place", "load_checkpoint", "random_tensors", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "model_files", "save_file"]

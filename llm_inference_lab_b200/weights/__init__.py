from .loader import WeightsError, check_folder, kept_dtype, load_weights
from .random_init import write_random_model
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, save_file

__all__ = ["WeightsError", "check_folder", "kept_dtype", "load_weights", "write_random_model",
           "ModelFiles", "SafetensorsError", "SafetensorsFile", "save_file"]

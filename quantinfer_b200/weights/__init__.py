from .loader import TensorNeed, check_and_load, load_folder
from .random_weights import random_tensors, write_model_folder
from .safetensors_io import SafeTensorsFile, SafeTensorsFolder, write_safetensors

__all__ = [
    "TensorNeed", "check_and_load", "load_folder", "random_tensors", "write_model_folder",
    "SafeTensorsFile", "SafeTensorsFolder", "write_safetensors",
]

from .loader import TensorRequest, WeightError, check_checkpoint, held_dtype, load_tensors
from .helix_file import HelixFile, HelixFileError, is_helix_file, write_helix_file
from .random_init import random_tensors, write_model_folder
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors
from .source import open_model

__all__ = [
    "Checkpoint", "HelixFile", "HelixFileError", "SafetensorsError", "SafetensorsFile", "TensorRequest", "WeightError",
    "check_checkpoint", "held_dtype", "is_helix_file", "load_tensors", "open_model", "random_tensors", "write_model_folder",
    "write_helix_file", "write_safetensors",
]

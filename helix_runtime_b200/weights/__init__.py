from .loader import TensorRequest, WeightError, check_checkpoint, held_dtype, load_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = [
    "Checkpoint", "SafetensorsError", "SafetensorsFile", "TensorRequest", "WeightError",
    "check_checkpoint", "held_dtype", "load_tensors", "random_tensors", "write_model_folder",
    "write_safetensors",
]

from .loader import CheckpointMismatch, TensorSpec, check_tensors, load_tensors, resolve_checkpoint
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsFile, save_safetensors

__all__ = [
    "CheckpointMismatch", "TensorSpec", "check_tensors", "load_tensors", "resolve_checkpoint",
    "random_tensor", "random_tensors", "write_model_folder", "SafetensorsFile", "save_safetensors",
]

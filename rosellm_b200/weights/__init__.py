from .loader import NamedParam, WeightError, match_tensors, read_safetensors, to_device_tensor
from .random_init import random_tensors, write_model_folder

__all__ = [
    "NamedParam",
    "WeightError",
    "match_tensors",
    "random_tensors",
    "read_safetensors",
    "to_device_tensor",
    "write_model_folder",
]

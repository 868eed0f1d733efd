from .loader import TensorDict, WeightError, bind, check, expected_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors

__all__ = ["TensorDict", "WeightError", "bind", "check", "expected_tensors", "random_tensors",
           "write_random_model", "Checkpoint", "SafetensorsError", "write_safetensors"]

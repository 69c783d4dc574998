from .safetensors_io import SafetensorsError, SafetensorsFolder, write_safetensors
from .loader import (WeightError, check_tensors, expected_tensors, load_weights,
                     random_tensors, write_random_model)

__all__ = ["SafetensorsError", "SafetensorsFolder", "write_safetensors", "WeightError",
           "check_tensors", "expected_tensors", "load_weights", "random_tensors",
           "write_random_model"]

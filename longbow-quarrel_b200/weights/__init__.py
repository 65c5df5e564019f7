from .loader import WeightsError, load_weights
from .random_init import random_tensor, random_weights, tensor_seed, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .spec import WeightSpec

__all__ = ["WeightsError", "load_weights", "random_tensor", "random_weights", "tensor_seed",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightSpec"]

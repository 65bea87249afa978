"""Weights: the safetensors container, loading by tensor name, and the random-weights mode."""
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import TensorSpec, WeightsError, load_tensors
from .random_init import random_tensor, tensor_seed, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "TensorSpec", "WeightsError",
           "load_tensors", "random_tensor", "tensor_seed", "write_random_model"]

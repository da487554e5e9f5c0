"""Weights: the safetensors container, loading by tensor name, and random model folders."""
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightError, TensorSpec, load_weights
from .random_init import write_random_model, random_tensor

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightError", "TensorSpec",
           "load_weights", "write_random_model", "random_tensor"]

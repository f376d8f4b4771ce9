"""Weights: safetensors by tensor name, and the seeded random mode."""

from .loader import ParamSpec, WeightError, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["ParamSpec", "SafetensorsError", "SafetensorsFile", "WeightError", "load_tensors",
           "random_tensors", "write_random_model", "write_safetensors"]

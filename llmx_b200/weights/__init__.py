"""Weights: safetensors by tensor name, the checks, and the random-weights mode."""
from .safetensors import SafetensorsError, SafetensorsFile, TensorDirectory, read_header, write_safetensors
from .spec import TensorSpec, WeightError
from .loader import check_tensors, stored
from .random_init import RandomSource, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "TensorDirectory", "read_header", "write_safetensors",
           "TensorSpec", "WeightError", "check_tensors", "stored", "RandomSource", "write_random_model"]

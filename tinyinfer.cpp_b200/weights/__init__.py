"""Weights: safetensors by tensor name, strict checks, and the random-weights mode."""
from .gguf import GgufError, GgufFile, write_gguf
from .loader import (WeightsError, check_tensors, load_gguf, load_model_weights,
                     load_model_weights_gguf, storage_dtype)
from .random_init import random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["GgufError", "GgufFile", "SafetensorsError", "SafetensorsFile", "WeightsError",
           "check_tensors", "load_gguf", "load_model_weights", "load_model_weights_gguf",
           "random_tensor", "storage_dtype", "write_gguf", "write_random_model",
           "write_safetensors"]

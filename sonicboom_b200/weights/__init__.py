"""Weights: safetensors files, binding by name, and the random-weights mode."""
from .loader import TensorRequest, WeightError, check, fetch, kept_dtype
from .random_init import RandomSource, write_random_model
from .safetensors_io import (SafetensorsDir, SafetensorsError, SafetensorsFile,
                             write_safetensors)

__all__ = ["TensorRequest", "WeightError", "check", "fetch", "kept_dtype", "RandomSource",
           "write_random_model", "SafetensorsDir", "SafetensorsError", "SafetensorsFile",
           "write_safetensors"]

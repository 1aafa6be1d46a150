"""Weights: safetensors I/O, loading by name, and the random-weights mode."""

from .loader import WeightsError, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, open_checkpoint, write_safetensors

__all__ = [
    "SafetensorsFile",
    "WeightsError",
    "load_weights",
    "open_checkpoint",
    "random_tensors",
    "write_random_model",
    "write_safetensors",
]

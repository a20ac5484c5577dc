"""Weights: safetensors by tensor name, and random weights from a configuration and a seed."""

from .loader import compare_with_checkpoint, load_model, load_tensors
from .random_init import random_model, random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsFile, write_safetensors

__all__ = [
    "Checkpoint", "SafetensorsFile", "write_safetensors", "load_model", "load_tensors",
    "compare_with_checkpoint", "random_model", "random_tensors", "write_random_model",
]

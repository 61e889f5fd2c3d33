"""Weights: safetensors container, checked loading by name, random-weights mode."""
from .loader import WeightError, checkpoint_files, load_checkpoint
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightError", "checkpoint_files", "load_checkpoint", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
